// Grouped MXFP8 expert contractions on the sm_100a tensor cores.
//
// One persistent, warp-specialised kernel template serves both projections:
//   warp 0      TMA producer: per 128-byte K slab, a [128 x 128B] tile of the
//               activation rows, a [BLOCK_N x 128B] tile of the expert's weight
//               rows (both 128B-swizzled) and their UE8M0 scale atoms (bulk copies)
//   warp 1      allocates TMEM and issues four tcgen05.mma.kind::mxf8f6f4.block_scale
//               (K = 32 each) per slab
//   warps 4..7  move each slab's UE8M0 scale atoms shared memory -> registers -> TMEM
//               (tcgen05.st, one TMEM lane quadrant per warp, one TMEM slot per pipeline
//               stage) so the tensor pipe never spends time on tcgen05.cp
//   warps 8..15 epilogue: two warps per TMEM lane quadrant, each thread pulls half of
//               its accumulator row into registers with tcgen05.ld, hands the TMEM
//               buffer back to the MMA warp at once, then works from registers
//               EPI 0: + bias, clamp, act(gate) * up in fp32, MXFP8 re-quantisation
//                      of the fp32 product (32 consecutive intermediates live in
//                      one thread), codes + scale atoms out
//               EPI 1: + bias, x routing affinity, bf16 rows out
// Tiles are (128 positions) x (BLOCK_N weight rows); a tile's expert comes from
// block_to_expert, padded / inactive tiles are skipped.  Tiles are enumerated
// expert by expert, weight tile by weight tile, position tile fastest, so the
// CTAs that run side by side read the same weight tile from L2 (a per-CTA
// prologue derives each expert's position-tile range from block_to_expert).
// Blocks run up to the first zero in `conditions`.  Every mbarrier wait is
// bounded: on expiry the kernel records a code in `status`, stops issuing work
// and tears down.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace b200moe {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 128;  // bytes (= e4m3 elements) per pipeline slab
constexpr int kGroupM = 16;
constexpr int kMaxExperts = 512;
constexpr int kThreads = 512;  // warp 0 producer, 1 MMA, 4-7 scale-factor movers, 8-15 epilogue (2, 3 idle)

struct GemmParams {
  const uint8_t* a_sf;
  const uint8_t* b_sf;
  int64_t b_sf_expert_stride;
  int b_row_atoms;  // scale atoms along the weight-row axis per expert
  const int32_t* block_to_expert;
  const int32_t* conditions;
  const int32_t* tile_flags;  // per 128-position tile: non-zero if it holds a real token (NULL = all)
  const int32_t* tpi;
  int hidden_rows, n_blocks, B, E;
  int m_tiles_total, n_tiles, k_blocks;
  int n_total;  // weight rows per expert
  const float* bias;
  int act;
  float gate_lo, gate_hi, up_lo, up_hi;
  uint8_t* m_codes;
  uint8_t* m_sf;
  int I;
  const void* aff;
  int aff_dtype;
  int aff_per_row;  // 0: table [rows, E] addressed tok*E + e; 1: vector [rows] addressed tok
  __nv_bfloat16* y_pos;
  int H_out;
  // expert parallelism: when row_src is set, row r of the result goes to row (row_src[r] & 0xffffff) of the buffer
  // peer_out[row_src[r] >> 24] (the GPU the token came from, over NVLink) instead of y_pos
  const int32_t* row_src;
  int64_t peer_rows;
  void* peer_out[8];
  int32_t* status;
  unsigned long long* clock_probe;  // optional: CTA 0 writes {SM cycles, nanoseconds} spent in the kernel
  const float* col_scale;  // dense (bf16) variant: per-expert, per-weight-row dequantisation factors [E, n_total]
                           // of fp8-row weights (NULL = none), applied to the accumulator before the bias
  int w_format;     // element format of the weight operand (B200MOE_W_*); activations are e4m3
  uint32_t b_tx;    // bytes one weight-tile copy reports to its mbarrier
  int early_successor;  // 1: let the next launch in the stream begin as soon as SMs free up (it touches other rows)
  int tile_filter;  // which position tiles a launch walks when experts are contiguous: 0 all, 1 (CTA-pair
                    // kernel) only pairs of two live tiles, 2 (single-CTA kernel) only the tile an expert with
                    // an odd number of live tiles has left over
  int wait_predecessor;  // 1: launched with programmatic stream serialisation behind a launch that signalled
                         // early; wait for that launch to finish before this grid may finish
};

// Per-CTA tile schedule, built once in shared memory.
struct Sched {
  int tile_start[kMaxExperts + 1];  // tiles before expert e (expert-aligned order)
  int mt_first[kMaxExperts];        // first 128-position tile of expert e
  int mt_count[kMaxExperts];        // its number of position tiles among the active blocks
  int runs[kMaxExperts];            // how many separate block runs expert e has (1 when sorted); after the
                                    // build, in left-over mode: the expert of left-over tile i
  int n_live[kMaxExperts];          // 1 + index (among the expert's tiles) of its last tile that holds a token
  int left_m[kMaxExperts];          // left-over mode: position tile of left-over i
  int n_left;                       // left-over mode: number of left-over tiles
  int n_full;                       // tiles [0, n_full) are whole; each later index is half (128 weight rows) of
                                    // one of the tiles that would not fill a last round of CTAs
  int n_active;                     // blocks before the first zero condition
  int contiguous;                   // every expert's blocks are adjacent
  int total;                        // number of tiles to walk
};

// `mg` = position tiles per scheduling unit (1, or 2 when a CTA pair shares a weight tile).
// `halves`: single-CTA launches with 256-row weight tiles may cut the tiles of a partly filled last round in two.
__device__ __forceinline__ void build_sched(const GemmParams& p, Sched& s, int mg, bool halves, int n_units) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int sub = p.B >> 7;
  if (tid == 0) { s.n_active = p.n_blocks; s.contiguous = 1; }
  for (int e = tid; e < p.E; e += nthr) { s.mt_first[e] = 0; s.mt_count[e] = 0; s.runs[e] = 0; }
  __syncthreads();
  if (p.conditions != nullptr)
    for (int b = tid; b < p.n_blocks; b += nthr)
      if (p.conditions[b] == 0) atomicMin(&s.n_active, b);
  __syncthreads();
  const int n_active = s.n_active;
  for (int b = tid; b < n_active; b += nthr) {
    const int e = p.block_to_expert[b];
    if (e < 0 || e >= p.E) continue;
    if (b == 0 || p.block_to_expert[b - 1] != e) {
      s.mt_first[e] = b * sub;
      if (atomicAdd(&s.runs[e], 1) > 0) s.contiguous = 0;
    }
    atomicAdd(&s.mt_count[e], sub);
  }
  __syncthreads();
  for (int e = tid; e < p.E; e += nthr) {
    int live = s.mt_count[e];
    if (p.tile_flags != nullptr)
      while (live > 0 && p.tile_flags[s.mt_first[e] + live - 1] == 0) --live;
    s.n_live[e] = live;
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, n_left = 0;
    const bool leftovers = s.contiguous && p.tile_filter == 2;
    for (int e = 0; e < p.E; ++e) {
      s.tile_start[e] = run;
      if (s.contiguous && p.tile_filter == 1) {
        run += (s.n_live[e] / 2) * p.n_tiles;                // full pairs only; the odd tile goes to the other launch
      } else if (leftovers) {
        if (s.n_live[e] & 1) { s.left_m[n_left] = s.mt_first[e] + s.n_live[e] - 1; s.runs[n_left] = e; ++n_left; }
      } else {
        run += ((s.mt_count[e] + mg - 1) / mg) * p.n_tiles;  // an odd tile count leaves the last pair half empty
      }
    }
    s.n_left = n_left;
    if (leftovers) run = n_left * p.n_tiles;
    if (!s.contiguous && p.tile_filter == 2) run = 0;        // scattered blocks: the pair launch does everything
    s.tile_start[p.E] = run;
    // scattered blocks: pairs stay inside a block when it holds an even number of tiles, else every tile is
    // a unit of its own (the pair's second CTA idles)
    const int units = (mg == 2 && (sub & 1)) ? p.m_tiles_total : p.m_tiles_total / mg;
    s.total = (s.contiguous || p.tile_filter == 2) ? run : units * p.n_tiles;
    s.n_full = s.total;
    if (halves && (s.contiguous || p.tile_filter == 2) && s.total >= 2 * n_units) {
      // whole rounds of n_units tiles keep their width; if the rest fits one round even when cut in two, cut it:
      // the last round then takes half as long
      const int whole = (s.total / n_units) * n_units, rest = s.total - whole;
      if (rest > 0 && 2 * rest <= n_units) { s.n_full = whole; s.total = whole + 2 * rest; }
    }
  }
  __syncthreads();
}

// m_tile is the first position tile of the unit; with mg == 2 the pair's CTAs take m_tile and m_tile + 1, and
// `second` says whether m_tile + 1 is a tile of the same expert that holds tokens (an expert with an odd number
// of tiles ends in a half-empty pair: its second CTA still supplies half of the weight tile but copies no
// activations and writes nothing).
// `part`: -1 for a whole weight tile, 0 / 1 for its first / second 128 rows (see Sched::n_full).
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const Sched& s, int tile, int mg, int& m_tile,
                                            int& n_tile, int& expert, int& second, int& part) {
  second = mg == 2 ? 1 : 0;
  part = -1;
  if (tile >= s.n_full) {
    part = (tile - s.n_full) & 1;
    tile = s.n_full + ((tile - s.n_full) >> 1);
  }
  if (s.contiguous && p.tile_filter == 2) {
    const int i = tile % s.n_left;
    m_tile = s.left_m[i];
    expert = s.runs[i];
    n_tile = tile / s.n_left;
    return true;
  }
  if (s.contiguous) {
    int lo = 0, hi = p.E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s.tile_start[mid] <= tile) lo = mid; else hi = mid;
    }
    expert = lo;
    const int local = tile - s.tile_start[lo];
    const int cnt = p.tile_filter == 1 ? s.n_live[lo] / 2 : (s.mt_count[lo] + mg - 1) / mg;
    const int idx = local % cnt;
    m_tile = s.mt_first[lo] + idx * mg;
    n_tile = local / cnt;
    if (mg == 2 && idx * 2 + 1 >= s.mt_count[lo]) second = 0;
  } else {
    const bool solo = mg == 2 && ((p.B >> 7) & 1);
    if (solo) { mg = 1; second = 0; }
    const int units = p.m_tiles_total / mg;
    const int per_group = kGroupM * p.n_tiles;
    const int g = tile / per_group;
    const int first_m = g * kGroupM;
    const int gs = min(kGroupM, units - first_m);
    const int within = tile - g * per_group;
    m_tile = (first_m + within % gs) * mg;
    n_tile = within / gs;
    const int block = m_tile / (p.B >> 7);
    if (block >= s.n_active) return false;
    expert = p.block_to_expert[block];
    if (expert < 0 || expert >= p.E) return false;
  }
  if (p.tile_flags != nullptr) {
    if (second && p.tile_flags[m_tile + 1] == 0) second = 0;
    if (p.tile_flags[m_tile] == 0 && !second) return false;
  }
  return true;
}

// Activation rows worth copying for a 128-position tile: tile_flags holds the number of leading rows that can
// carry a token (tokens fill a block from its start), so short tiles -- decode, the last block of an expert --
// copy a 32- or 64-row box.  The MMA still spans 128 rows; what it computes from the stale rows below the box
// lands in rows nobody reads.
__device__ __forceinline__ int tile_copy_rows(const GemmParams& p, int m_tile) {
  if (p.tile_flags == nullptr) return kBlockM;
  const int f = p.tile_flags[m_tile];
  return f <= 0 ? 0 : (f <= 32 ? 32 : (f <= 64 ? 64 : kBlockM));
}

// A CTA's own tiles, decoded once in the prologue by all threads: the per-tile decode (a search over the experts,
// two divisions, tile_flags reads from global memory) costs about a thousand clocks, which the single MMA-issuing
// thread would otherwise spend at every tile boundary with the tensor pipe idle.
struct TileRec {
  int m_tile, n_tile, expert;
  int flags;  // bit 0 valid, bit 1 second, bits 2-3 part + 1, bits 8-15 / 16-23 activation rows to copy (lead / peer)
};
constexpr int kTileTable = 448;  // entries per CTA (7 KB); later tiles are decoded on the spot

__device__ __forceinline__ bool fetch_tile(const GemmParams& p, const Sched& s, const TileRec* table, int it, int tile,
                                           int mg, int& m_tile, int& n_tile, int& expert, int& second, int& part,
                                           int& rows_lead, int& rows_peer) {
  if (it < kTileTable) {
    const int4 r = *reinterpret_cast<const int4*>(table + it);
    if (!(r.w & 1)) return false;
    m_tile = r.x;
    n_tile = r.y;
    expert = r.z;
    second = (r.w >> 1) & 1;
    part = ((r.w >> 2) & 3) - 1;
    rows_lead = (r.w >> 8) & 0xff;
    rows_peer = (r.w >> 16) & 0xff;
    return true;
  }
  if (!decode_tile(p, s, tile, mg, m_tile, n_tile, expert, second, part)) return false;
  rows_lead = tile_copy_rows(p, m_tile);
  rows_peer = second ? tile_copy_rows(p, m_tile + 1) : 0;
  return true;
}

template <int BLOCK_N, int STAGES, int CTAS = 1>
struct SmemLayout {
  static constexpr int kA = kBlockM * kBlockK;
  static constexpr int kB = (BLOCK_N / CTAS) * kBlockK;  // a CTA pair splits the weight rows
  static constexpr int kSfa = 512;
  static constexpr int kSfbAtoms = BLOCK_N > 128 ? 2 : 1;
  static constexpr int kSfb = kSfbAtoms * 512;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + STAGES * kA;
  static constexpr int kOffSfa = kOffB + STAGES * kB;
  static constexpr int kOffSfb = kOffSfa + STAGES * kSfa;
  static constexpr int kOffBar = kOffSfb + STAGES * kSfb;
  static constexpr int kOffSched = kOffBar + 256;
  static constexpr int kOffTiles = (kOffSched + static_cast<int>(sizeof(Sched)) + 15) & ~15;
  static constexpr int kBytes = kOffTiles + kTileTable * static_cast<int>(sizeof(TileRec)) + 1024;  // + alignment slack
};

// KIND 0: MXFP8 activations x MX weights, block-scaled MMAs (kind::mxf8f6f4.block_scale).
// KIND 1: bf16 activations x bf16 weights (kind::f16), the reference's non-MX variants: no scale atoms travel, the
//         four scale-mover warps idle, the gate/up epilogue writes bf16 intermediates instead of MX codes.  Operand
//         rows are addressed in bytes, so a 128-byte slab is 64 bf16 elements = four K = 16 MMAs.
template <int BLOCK_N, int STAGES, int EPI, int CTAS, int KIND = 0>
__global__ void __launch_bounds__(kThreads, 1)
grouped_mxfp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a64,
                          const __grid_constant__ CUtensorMap tmap_a32, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_b128, const __grid_constant__ CUtensorMap tmap_sfa,
                          const __grid_constant__ CUtensorMap tmap_sfb, const GemmParams p) {
  // CTAS == 2: the two CTAs of a cluster form one tcgen05 cta_group::2 unit.  Each loads its own 128
  // activation rows and half of the weight tile; the even CTA issues M = 256 MMAs that read both CTAs'
  // shared memory and write both CTAs' TMEM, so a weight byte crosses L2 -> SM once per 256 rows.
  using L = SmemLayout<BLOCK_N, STAGES, CTAS>;
  constexpr int kAcc = (BLOCK_N <= 128) ? 2 : 1;
  constexpr int kSfCol = kAcc * BLOCK_N;  // TMEM columns: accumulators, then SFA (4), then SFB
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdesc = KIND == 0 ? make_idesc(kBlockM * CTAS, BLOCK_N) : make_idesc_bf16(kBlockM * CTAS, BLOCK_N);
  // operand bytes per stage (scale atoms report to sf_full) depend on the tile: short activation boxes, and
  // 4-bit weights that land in the same padded 128-byte rows but report their packed size
  const uint32_t idesc_base = KIND == 0 ? (kIdesc | (static_cast<uint32_t>(p.w_format) << 10)) : kIdesc;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + kAcc;
  uint64_t* sf_full = bars + 2 * STAGES + 2 * kAcc;             // scale atoms of a stage landed (per CTA)
  uint64_t* sf_ready = bars + 3 * STAGES + 2 * kAcc;            // ... and sit in their TMEM slot (pair leader)
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 4 * STAGES + 2 * kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  Sched& sched = *reinterpret_cast<Sched*>(smem + L::kOffSched);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long probe_c0 = 0;
  unsigned long long probe_t0 = 0;
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    probe_c0 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(probe_t0));
  }
  // The left-over launch that follows a CTA-pair launch works on different rows of the same buffers: it may start
  // on every SM this launch no longer needs (programmatic dependent launch).  The successor does its tiles without
  // waiting and executes griddepcontrol.wait before it exits, so it never completes before this grid has.
  if (p.early_successor && threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int cta_rank = CTAS == 2 ? static_cast<int>(cluster_cta_rank()) : 0;
  const int unit = blockIdx.x / CTAS, n_units = gridDim.x / CTAS;
  build_sched(p, sched, CTAS, CTAS == 1 && BLOCK_N == 256, n_units);
  const int total_tiles = sched.total;
  TileRec* tile_table = reinterpret_cast<TileRec*>(smem + L::kOffTiles);
  for (int i = threadIdx.x; i < kTileTable; i += kThreads) {
    const int tile = unit + i * n_units;
    TileRec r{0, 0, 0, 0};
    if (tile < total_tiles) {
      int m_tile, n_tile, e, second, part;
      if (decode_tile(p, sched, tile, CTAS, m_tile, n_tile, e, second, part)) {
        const int rl = tile_copy_rows(p, m_tile), rp = second ? tile_copy_rows(p, m_tile + 1) : 0;
        r = TileRec{m_tile, n_tile, e, 1 | (second << 1) | ((part + 1) << 2) | (rl << 8) | (rp << 16)};
      }
    }
    tile_table[i] = r;  // read after the __syncthreads below
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&sf_full[s], 1);
      mbar_init(&sf_ready[s], 4 * CTAS);
    }
    for (int a = 0; a < kAcc; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8 * CTAS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  // Register budget per warpgroup (4 warps): the epilogue warps hold 128 accumulator values per thread,
  // everyone else needs few.  512 threads x 128 at launch = 2 x 128 x 64 + 2 x 128 x 192.
  if (warp < 4) {
    reg_dec<64>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      constexpr int kRowsB = BLOCK_N / CTAS;  // weight rows this CTA copies per slab
      for (int tile = unit, it = 0; tile < total_tiles && ok; tile += n_units, ++it) {
        int m_tile, n_tile, e, second, part, rows_lead, rows_peer;
        if (!fetch_tile(p, sched, tile_table, it, tile, CTAS, m_tile, n_tile, e, second, part, rows_lead, rows_peer))
          continue;
        m_tile += cta_rank;
        const int my_rows = cta_rank == 0 ? rows_lead : rows_peer;
        const CUtensorMap* map_a = my_rows == 32 ? &tmap_a32 : (my_rows == 64 ? &tmap_a64 : &tmap_a);
        // a half tile (single-CTA launches only) copies 128 weight rows through the 128-row map
        const int n_row0 = n_tile * BLOCK_N + (part > 0 ? BLOCK_N / 2 : 0);
        const uint32_t b_bytes = part >= 0 ? p.b_tx / 2 : p.b_tx;
        const uint32_t stage_bytes = static_cast<uint32_t>(rows_lead + rows_peer) * kBlockK + CTAS * b_bytes;
        const int atom0 = n_row0 >> 7;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          // scale atoms of this CTA's rows and of the whole weight tile -> this CTA's own barrier
          // (rows past the end of the atom table read as zero and still count their bytes)
          if constexpr (KIND == 0) {
            mbar_expect_tx(&sf_full[stage], L::kSfa + L::kSfb);
            tma_load_2d(smem + L::kOffSfa + stage * L::kSfa, &tmap_sfa, 0, m_tile * p.k_blocks + kb, &sf_full[stage]);
#pragma unroll
            for (int j = 0; j < L::kSfbAtoms; ++j)
              tma_load_2d(smem + L::kOffSfb + stage * L::kSfb + j * 512, &tmap_sfb, 0,
                          (e * p.b_row_atoms + atom0 + j) * p.k_blocks + kb, &sf_full[stage]);
          }
          if constexpr (CTAS == 2) {
            // operand tiles of both CTAs complete on the even CTA's barrier
            if (cta_rank == 0) mbar_expect_tx(&full[stage], stage_bytes);
            if (my_rows > 0)
              tma2_load_2d(smem + L::kOffA + stage * L::kA, map_a, kb * kBlockK, m_tile * kBlockM, &full[stage]);
            tma2_load_3d(smem + L::kOffB + stage * L::kB, &tmap_b, kb * kBlockK,
                         n_tile * BLOCK_N + cta_rank * (BLOCK_N / 2), e, &full[stage]);
          } else {
            mbar_expect_tx(&full[stage], stage_bytes);
            if (my_rows > 0)
              tma_load_2d(smem + L::kOffA + stage * L::kA, map_a, kb * kBlockK, m_tile * kBlockM, &full[stage]);
            tma_load_3d(smem + L::kOffB + stage * L::kB, part >= 0 ? &tmap_b128 : &tmap_b, kb * kBlockK, n_row0, e,
                        &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let copies already in flight land before the CTA retires
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only when paired)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = unit, it = 0; tile < total_tiles && ok; tile += n_units, ++it) {
        int m_tile, n_tile, e, second, part, rows_lead, rows_peer;
        if (!fetch_tile(p, sched, tile_table, it, tile, CTAS, m_tile, n_tile, e, second, part, rows_lead, rows_peer))
          continue;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        const int n_row0 = n_tile * BLOCK_N + (part > 0 ? BLOCK_N / 2 : 0);
        const uint32_t sfb_off = (n_row0 & 127) >> 5;  // a tile may start mid-atom
        // half tiles run N = 128 MMAs into the first 128 accumulator columns
        const uint32_t idesc_tile = part >= 0 ? ((idesc_base & ~(0x3Fu << 17)) | (static_cast<uint32_t>(128 >> 3) << 17))
                                              : idesc_base;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
          if constexpr (KIND == 0)
            if (!mbar_wait(&sf_ready[stage], phase, abort_flag, p.status, 5)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sfa_tmem = tmem_base + kSfCol + stage * 16;
          const uint32_t sfb_tmem = sfa_tmem + 4 + sfb_off;
          const uint64_t a_desc = desc_sw128(smem_u32(smem + L::kOffA + stage * L::kA));
          const uint64_t b_desc = desc_sw128(smem_u32(smem + L::kOffB + stage * L::kB));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if constexpr (KIND == 0) {
              const uint32_t idesc = idesc_tile | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
              if constexpr (CTAS == 2)
                tc2_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa_tmem, sfb_tmem, (kb | k) != 0 ? 1u : 0u);
              else
                tc_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa_tmem, sfb_tmem, (kb | k) != 0 ? 1u : 0u);
            } else {
              if constexpr (CTAS == 2) tc2_mma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_tile, (kb | k) != 0 ? 1u : 0u);
              else tc_mma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_tile, (kb | k) != 0 ? 1u : 0u);
            }
          }
          if constexpr (CTAS == 2) tc2_commit_pair(&empty[stage]);
          else tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if constexpr (CTAS == 2) tc2_commit_pair(&tmem_full[acc]);
          else tc_commit(&tmem_full[acc]);
        }
        if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
      }
    }
  }
  } else if (warp < 8) {
    reg_dec<64>();
    // ------------------------------------------------------------ scale-factor movers (one TMEM lane quadrant each)
    // Lane l of a quadrant owns rows l, l+32, l+64, l+96 of every atom: the 16 bytes at l*16 are the four
    // 32-bit TMEM cells (4 scale bytes each) the block-scaled MMA expects in that lane.
    const int q = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = unit, it = 0; KIND == 0 && tile < total_tiles && ok; tile += n_units, ++it) {
      int m_tile, n_tile, e, second, part, rows_lead, rows_peer;
      if (!fetch_tile(p, sched, tile_table, it, tile, CTAS, m_tile, n_tile, e, second, part, rows_lead, rows_peer))
        continue;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(&sf_full[stage], phase, abort_flag, p.status, 6)) { ok = false; break; }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kSfCol + stage * 16;
        {
          const uint4 va = *reinterpret_cast<const uint4*>(smem + L::kOffSfa + stage * L::kSfa + lane * 16);
          tc_st4(taddr, va);
#pragma unroll
          for (int j = 0; j < L::kSfbAtoms; ++j) {
            const uint4 vb = *reinterpret_cast<const uint4*>(smem + L::kOffSfb + stage * L::kSfb + j * 512 + lane * 16);
            tc_st4(taddr + 4 + 4 * j, vb);
          }
          tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTAS == 2 && cta_rank != 0) mbar_arrive_leader_relaxed(&sf_ready[stage]);
          else mbar_arrive(&sf_ready[stage]);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    reg_inc<192>();
    // ------------------------------------------------------------ epilogue (every CTA drains its own TMEM)
    constexpr int kCW = BLOCK_N / 2;   // accumulator columns per thread
    constexpr int kLd = kCW / 32;      // 32-column TMEM loads per thread
    const int q = warp & 3;
    const int half = (warp - 8) >> 2;
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool clamp = (p.gate_lo == p.gate_lo) || (p.gate_hi == p.gate_hi) || (p.up_lo == p.up_lo) ||
                       (p.up_hi == p.up_hi);
    const float g_lo = p.gate_lo == p.gate_lo ? p.gate_lo : -INFINITY, g_hi = p.gate_hi == p.gate_hi ? p.gate_hi : INFINITY;
    const float u_lo = p.up_lo == p.up_lo ? p.up_lo : -INFINITY, u_hi = p.up_hi == p.up_hi ? p.up_hi : INFINITY;
    for (int tile = unit, it = 0; tile < total_tiles; tile += n_units, ++it) {
      int m_tile, n_tile, e, second, part, rows_lead, rows_peer;
      if (!fetch_tile(p, sched, tile_table, it, tile, CTAS, m_tile, n_tile, e, second, part, rows_lead, rows_peer))
        continue;
      m_tile += cta_rank;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, 4)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N + half * kCW;
      const int64_t row = static_cast<int64_t>(m_tile) * kBlockM + row_in_tile;
      uint32_t raw[kLd][32];
#pragma unroll
      for (int l = 0; l < kLd; ++l) tc_ld32_nowait(taddr + l * 32, raw[l]);
      tc_wait_ld();
      // the accumulator now lives in registers: give the TMEM buffer back before doing the math
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        // relaxed: the accumulator is in registers (wait::ld above); a releasing arrive would first wait for this
        // thread's global stores of the previous tile to become visible and hold the next tile's MMAs back
        if (CTAS == 2 && cta_rank != 0) mbar_arrive_leader_relaxed(&tmem_empty[acc]);
        else mbar_arrive_relaxed(&tmem_empty[acc]);
      }
      if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
      if (CTAS == 2 && cta_rank != 0 && !second) continue;  // half-empty pair: these rows belong to someone else
      if (part >= 0 && half != 0) continue;                 // half tile: only 128 accumulator columns hold results
      const int n_row0 = n_tile * BLOCK_N + (part > 0 ? BLOCK_N / 2 : 0);

      if constexpr (EPI == 0) {
        const int64_t k_atoms = (p.I + 127) >> 7;
        const float* bias = p.bias ? p.bias + static_cast<int64_t>(e) * p.n_total : nullptr;
#pragma unroll
        for (int c = 0; c < kLd / 2; ++c) {
          const int n0 = n_row0 + half * kCW + c * 64;
          const int i0 = n0 >> 1;
          if (i0 >= p.I) continue;
          float g[32], u[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) { g[j] = __uint_as_float(raw[2 * c][j]); u[j] = __uint_as_float(raw[2 * c + 1][j]); }
          if constexpr (KIND == 1) {
            if (p.col_scale != nullptr) {
              const float* cs = p.col_scale + static_cast<int64_t>(e) * p.n_total + n0;
#pragma unroll
              for (int j = 0; j < 32; ++j) { g[j] *= cs[j]; u[j] *= cs[32 + j]; }
            }
          }
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) { g[j] += bias[n0 + j]; u[j] += bias[n0 + 32 + j]; }
          }
          if (clamp) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              g[j] = fminf(fmaxf(g[j], g_lo), g_hi);
              u[j] = fminf(fmaxf(u[j], u_lo), u_hi);
            }
          }
          uint32_t mx = 0;
          if (p.act == B200MOE_ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float sg = __fdividef(g[j], 1.0f + __expf(-g[j]));
              const float m = sg * u[j];
              g[j] = m;
              mx = max(mx, __float_as_uint(m) & 0x7fffffffu);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float m = apply_act(g[j], p.act) * u[j];
              g[j] = m;
              mx = max(mx, __float_as_uint(m) & 0x7fffffffu);
            }
          }
          if constexpr (KIND == 1) {
            // dense variant: the intermediate stays bf16 (the next contraction's operand type)
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(g[2 * j], g[2 * j + 1]);
              o[j] = *reinterpret_cast<const uint32_t*>(&b2);
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.m_codes) + row * p.I + i0;
            st_global_256(dst, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
            st_global_256(dst + 16, o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]);
            continue;
          }
          uint32_t w[8];
          const int e_max = static_cast<int>(mx >> 23);
          if (e_max >= 9) {  // one exact power-of-two factor
            const float f = __uint_as_float(static_cast<uint32_t>(135 - e_max + 127) << 23);
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = pack4_e4m3(g[4 * j] * f, g[4 * j + 1] * f, g[4 * j + 2] * f, g[4 * j + 3] * f);
          } else {
            float f1, f2;
            mx_block_factors(mx, f1, f2);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              w[j] = pack4_e4m3(g[4 * j] * f1 * f2, g[4 * j + 1] * f1 * f2, g[4 * j + 2] * f1 * f2, g[4 * j + 3] * f1 * f2);
          }
          st_global_256(p.m_codes + row * p.I + i0, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
          p.m_sf[sf_atom_offset(row, i0 >> 5, k_atoms)] = mx_block_scale_byte(mx);
        }
      } else {
        const int tok = p.tpi ? p.tpi[row] : static_cast<int>(row);
        bool valid = tok >= 0 && tok < p.hidden_rows;
        __nv_bfloat16* out_row = p.y_pos + row * p.H_out;
        if (p.row_src != nullptr && valid) {
          const int32_t src = p.row_src[row];
          const int dst_rank = (src >> 24) & 0x7f;
          const int64_t dst_row = src & 0xffffff;
          valid = dst_rank < 8 && dst_row < p.peer_rows && p.peer_out[dst_rank] != nullptr;
          if (valid) out_row = static_cast<__nv_bfloat16*>(p.peer_out[dst_rank]) + dst_row * p.H_out;
        }
        float aff = 1.0f;
        if (valid && p.aff != nullptr)
          aff = load_as_float(p.aff, p.aff_per_row ? static_cast<int64_t>(tok) : static_cast<int64_t>(tok) * p.E + e,
                              p.aff_dtype);
        const float* bias = p.bias ? p.bias + static_cast<int64_t>(e) * p.H_out : nullptr;
        const float* cs = (KIND == 1 && p.col_scale) ? p.col_scale + static_cast<int64_t>(e) * p.H_out : nullptr;
#pragma unroll
        for (int l = 0; l < kLd; ++l) {
          const int col0 = n_row0 + half * kCW + l * 32;
          if (col0 >= p.H_out || !valid) continue;
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float a0 = __uint_as_float(raw[l][2 * j]), a1 = __uint_as_float(raw[l][2 * j + 1]);
            if (cs) { a0 *= cs[col0 + 2 * j]; a1 *= cs[col0 + 2 * j + 1]; }
            if (bias) { a0 += bias[col0 + 2 * j]; a1 += bias[col0 + 2 * j + 1]; }
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(a0 * aff, a1 * aff);
            o[j] = *reinterpret_cast<const uint32_t*>(&b2);
          }
#pragma unroll
          for (int j = 0; j < 2; ++j)
            st_global_256(out_row + col0 + 16 * j, o[8 * j], o[8 * j + 1], o[8 * j + 2], o[8 * j + 3], o[8 * j + 4],
                          o[8 * j + 5], o[8 * j + 6], o[8 * j + 7]);
        }
      }
    }
  }

  // A grid that was allowed to start while its predecessor drains must not finish before it: whatever follows in
  // the stream waits for this grid only, and relies on both having completed.
  if (p.wait_predecessor) asm volatile("griddepcontrol.wait;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    p.clock_probe[0] = static_cast<unsigned long long>(clock64() - probe_c0);
    p.clock_probe[1] = t1 - probe_t0;
  }
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer may still read this CTA's shared memory until here
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CTAS == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ validation kernels (CUDA cores)
__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ int64_t weight_offset(int64_t rows, int K, int w_format) {
  return w_format == B200MOE_W_E2M1 ? rows * K / 2 : rows * K;
}
// Weight element k of a row of K elements in any of the supported formats.
__device__ __forceinline__ float weight_to_float(const uint8_t* row, int k, int w_format) {
  if (w_format == B200MOE_W_E2M1) {
    const uint32_t nib = (row[k >> 1] >> ((k & 1) * 4)) & 0xFu;
    const uint32_t ex = (nib >> 1) & 3u, man = nib & 1u;
    const float mag = ex == 0 ? 0.5f * man : (1.0f + 0.5f * man) * static_cast<float>(1u << (ex - 1));
    return (nib & 8u) ? -mag : mag;
  }
  if (w_format == B200MOE_W_E5M2) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(row[k]), __NV_E5M2);
    return __half2float(*reinterpret_cast<const __half*>(&h));
  }
  return e4m3_to_float(row[k]);
}

__device__ float mx_dot(const uint8_t* a, const uint8_t* a_sf, int64_t a_row, const uint8_t* b, const uint8_t* b_sf,
                        int64_t b_row, int K, int w_format) {
  const int64_t k_atoms = (K + 127) >> 7;
  const uint8_t* brow = b + b_row * (w_format == B200MOE_W_E2M1 ? K / 2 : K);
  float acc = 0.f;
  for (int kb = 0; kb < K / 32; ++kb) {
    float part = 0.f;
    for (int j = 0; j < 32; ++j)
      part += e4m3_to_float(a[a_row * K + kb * 32 + j]) * weight_to_float(brow, kb * 32 + j, w_format);
    const int sa = a_sf[sf_atom_offset(a_row, kb, k_atoms)], sb = b_sf[sf_atom_offset(b_row, kb, k_atoms)];
    acc += part * exp2f(static_cast<float>(sa - 127)) * exp2f(static_cast<float>(sb - 127));
  }
  return acc;
}

__device__ bool block_is_active(const GemmParams& p, int block) {
  if (p.conditions == nullptr) return true;
  for (int b = 0; b <= block; ++b)
    if (p.conditions[b] == 0) return false;
  return true;
}

__global__ void simt_gemm1_kernel(const uint8_t* x, const uint8_t* w, GemmParams p, int K) {
  // one thread per (position, 32-block of intermediates)
  const int blocks_i = p.I / 32;
  const int64_t total = static_cast<int64_t>(p.m_tiles_total) * 128 * blocks_i;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int ib = static_cast<int>(idx % blocks_i);
    const int64_t row = idx / blocks_i;
    const int m_tile = static_cast<int>(row >> 7);
    const int block = m_tile / (p.B >> 7);
    if (!block_is_active(p, block)) continue;
    if (p.tile_flags && p.tile_flags[m_tile] == 0) continue;
    const int e = p.block_to_expert[block];
    if (e < 0 || e >= p.E) continue;
    const uint8_t* we = w + weight_offset(static_cast<int64_t>(e) * p.n_total, K, p.w_format);
    const uint8_t* wsf = p.b_sf + static_cast<int64_t>(e) * p.b_sf_expert_stride;
    const float* bias = p.bias ? p.bias + static_cast<int64_t>(e) * p.n_total : nullptr;
    float m[32];
    uint32_t mx = 0;
    for (int j = 0; j < 32; ++j) {
      const int n_g = ib * 64 + j, n_u = n_g + 32;
      float gv = mx_dot(x, p.a_sf, row, we, wsf, n_g, K, p.w_format);
      float uv = mx_dot(x, p.a_sf, row, we, wsf, n_u, K, p.w_format);
      if (bias) { gv += bias[n_g]; uv += bias[n_u]; }
      if (p.gate_lo == p.gate_lo) gv = fmaxf(gv, p.gate_lo);
      if (p.gate_hi == p.gate_hi) gv = fminf(gv, p.gate_hi);
      if (p.up_lo == p.up_lo) uv = fmaxf(uv, p.up_lo);
      if (p.up_hi == p.up_hi) uv = fminf(uv, p.up_hi);
      m[j] = apply_act(gv, p.act) * uv;
      mx = max(mx, __float_as_uint(m[j]) & 0x7fffffffu);
    }
    float f1, f2;
    mx_block_factors(mx, f1, f2);
    uint32_t* dst = reinterpret_cast<uint32_t*>(p.m_codes + row * p.I + ib * 32);
    for (int j = 0; j < 8; ++j)
      dst[j] = pack4_e4m3(m[4 * j] * f1 * f2, m[4 * j + 1] * f1 * f2, m[4 * j + 2] * f1 * f2, m[4 * j + 3] * f1 * f2);
    p.m_sf[sf_atom_offset(row, ib, (p.I + 127) >> 7)] = mx_block_scale_byte(mx);
  }
}

__global__ void simt_gemm2_kernel(const uint8_t* m, const uint8_t* w, GemmParams p, int K) {
  const int64_t total = static_cast<int64_t>(p.m_tiles_total) * 128 * p.H_out;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int h = static_cast<int>(idx % p.H_out);
    const int64_t row = idx / p.H_out;
    const int m_tile = static_cast<int>(row >> 7);
    const int block = m_tile / (p.B >> 7);
    if (!block_is_active(p, block)) continue;
    if (p.tile_flags && p.tile_flags[m_tile] == 0) continue;
    const int e = p.block_to_expert[block];
    if (e < 0 || e >= p.E) continue;
    const int tok = p.tpi ? p.tpi[row] : static_cast<int>(row);
    if (tok < 0 || tok >= p.hidden_rows) continue;
    float y = mx_dot(m, p.a_sf, row, w + weight_offset(static_cast<int64_t>(e) * p.n_total, K, p.w_format),
                     p.b_sf + static_cast<int64_t>(e) * p.b_sf_expert_stride, h, K, p.w_format);
    if (p.bias) y += p.bias[static_cast<int64_t>(e) * p.H_out + h];
    if (p.aff)
      y *= load_as_float(p.aff, p.aff_per_row ? static_cast<int64_t>(tok) : static_cast<int64_t>(tok) * p.E + e,
                         p.aff_dtype);
    __nv_bfloat16* out_row = p.y_pos + row * p.H_out;
    if (p.row_src != nullptr) {
      const int32_t src = p.row_src[row];
      const int dst_rank = (src >> 24) & 0x7f;
      const int64_t dst_row = src & 0xffffff;
      if (dst_rank >= 8 || dst_row >= p.peer_rows || p.peer_out[dst_rank] == nullptr) continue;
      out_row = static_cast<__nv_bfloat16*>(p.peer_out[dst_rank]) + dst_row * p.H_out;
    }
    out_row[h] = __float2bfloat16_rn(y);
  }
}

// Dense (bf16 x bf16) counterparts of the two validation kernels: one thread per output element.
__device__ float dense_dot(const __nv_bfloat16* a, const __nv_bfloat16* b, int K) {
  float acc = 0.f;
  for (int k = 0; k < K; ++k) acc += __bfloat162float(a[k]) * __bfloat162float(b[k]);
  return acc;
}

__global__ void simt_dense_gemm1_kernel(const __nv_bfloat16* x, const __nv_bfloat16* w, GemmParams p, int K) {
  const int64_t total = static_cast<int64_t>(p.m_tiles_total) * 128 * p.I;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % p.I);
    const int64_t row = idx / p.I;
    const int m_tile = static_cast<int>(row >> 7);
    const int block = m_tile / (p.B >> 7);
    if (!block_is_active(p, block)) continue;
    if (p.tile_flags && p.tile_flags[m_tile] == 0) continue;
    const int e = p.block_to_expert[block];
    if (e < 0 || e >= p.E) continue;
    const int n_g = (i >> 5) * 64 + (i & 31), n_u = n_g + 32;
    const __nv_bfloat16* we = w + static_cast<int64_t>(e) * p.n_total * K;
    float gv = dense_dot(x + row * K, we + static_cast<int64_t>(n_g) * K, K);
    float uv = dense_dot(x + row * K, we + static_cast<int64_t>(n_u) * K, K);
    if (p.col_scale) {
      gv *= p.col_scale[static_cast<int64_t>(e) * p.n_total + n_g];
      uv *= p.col_scale[static_cast<int64_t>(e) * p.n_total + n_u];
    }
    if (p.bias) { gv += p.bias[static_cast<int64_t>(e) * p.n_total + n_g]; uv += p.bias[static_cast<int64_t>(e) * p.n_total + n_u]; }
    if (p.gate_lo == p.gate_lo) gv = fmaxf(gv, p.gate_lo);
    if (p.gate_hi == p.gate_hi) gv = fminf(gv, p.gate_hi);
    if (p.up_lo == p.up_lo) uv = fmaxf(uv, p.up_lo);
    if (p.up_hi == p.up_hi) uv = fminf(uv, p.up_hi);
    reinterpret_cast<__nv_bfloat16*>(p.m_codes)[row * p.I + i] = __float2bfloat16_rn(apply_act(gv, p.act) * uv);
  }
}

__global__ void simt_dense_gemm2_kernel(const __nv_bfloat16* m, const __nv_bfloat16* w, GemmParams p, int K) {
  const int64_t total = static_cast<int64_t>(p.m_tiles_total) * 128 * p.H_out;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int h = static_cast<int>(idx % p.H_out);
    const int64_t row = idx / p.H_out;
    const int m_tile = static_cast<int>(row >> 7);
    const int block = m_tile / (p.B >> 7);
    if (!block_is_active(p, block)) continue;
    if (p.tile_flags && p.tile_flags[m_tile] == 0) continue;
    const int e = p.block_to_expert[block];
    if (e < 0 || e >= p.E) continue;
    const int tok = p.tpi ? p.tpi[row] : static_cast<int>(row);
    if (tok < 0 || tok >= p.hidden_rows) continue;
    float y = dense_dot(m + row * K, w + (static_cast<int64_t>(e) * p.n_total + h) * K, K);
    if (p.col_scale) y *= p.col_scale[static_cast<int64_t>(e) * p.H_out + h];
    if (p.bias) y += p.bias[static_cast<int64_t>(e) * p.H_out + h];
    if (p.aff)
      y *= load_as_float(p.aff, p.aff_per_row ? static_cast<int64_t>(tok) : static_cast<int64_t>(tok) * p.E + e,
                         p.aff_dtype);
    p.y_pos[row * p.H_out + h] = __float2bfloat16_rn(y);
  }
}

// ------------------------------------------------------------------ host side
// Rows of K elements, one byte each, or (nibbles) two per byte: the 4-bit map type expands every 8 packed
// bytes to a 16-byte shared-memory chunk, which is the padded form the f8f6f4 MMA reads 4-bit operands in,
// so a 128-element slab still occupies a 128-byte swizzled row.
int make_rows_map(CUtensorMap* map, const void* base, int64_t K, int64_t rows, int64_t batch, int box_rows,
                  bool nibbles = false) {
  EncodeTiledFn enc = get_encode_fn();
  B200MOE_REQUIRE(enc != nullptr, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint32_t rank = batch > 0 ? 3 : 2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch > 0 ? batch : 1)};
  const cuuint64_t pitch = static_cast<cuuint64_t>(nibbles ? K / 2 : K);
  cuuint64_t strides[2] = {pitch, pitch * static_cast<cuuint64_t>(rows)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, nibbles ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, rank,
                         const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200MOE_REQUIRE(r == CUDA_SUCCESS, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return B200MOE_OK;
}

int make_atoms_map(CUtensorMap* map, const void* base, int64_t n_atoms) {
  // scale atoms as rows of 128 32-bit words, one atom per TMA box
  EncodeTiledFn enc = get_encode_fn();
  B200MOE_REQUIRE(enc != nullptr, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(n_atoms)};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200MOE_REQUIRE(r == CUDA_SUCCESS, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled (scale atoms) failed with code %d",
                  static_cast<int>(r));
  return B200MOE_OK;
}

template <int BLOCK_N, int STAGES, int EPI, int CTAS, int KIND = 0>
int launch_tc(const CUtensorMap (&ma)[3], const CUtensorMap& mb, const CUtensorMap& mb128, const CUtensorMap& msa,
              const CUtensorMap& msb, const GemmParams& p, cudaStream_t st, bool overlap_predecessor = false) {
  using L = SmemLayout<BLOCK_N, STAGES, CTAS>;
  auto kern = grouped_mxfp8_gemm_kernel<BLOCK_N, STAGES, EPI, CTAS, KIND>;
  B200MOE_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kBytes));
  // only sizes the grid; a left-over launch has at most one tile per expert and weight tile
  const int total = p.tile_filter == 2 ? p.E * p.n_tiles : ((p.m_tiles_total + CTAS - 1) / CTAS) * p.n_tiles;
  int grid = (total < sm_count() / CTAS ? total : sm_count() / CTAS) * CTAS;
  if constexpr (CTAS == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200MOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ma[0], ma[1], ma[2], mb, mb128, msa, msb, p));
  } else if (overlap_predecessor) {
    // programmatic stream serialisation: this grid may be scheduled while the previous kernel of the stream is
    // still draining (the kernel never waits for it: it shares no rows with it)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200MOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ma[0], ma[1], ma[2], mb, mb128, msa, msb, p));
  } else {
    kern<<<grid, kThreads, L::kBytes, st>>>(ma[0], ma[1], ma[2], mb, mb128, msa, msb, p);
  }
  B200MOE_LAUNCH_OK("grouped_mxfp8_gemm_kernel");
  return B200MOE_OK;
}

// `impl` is the per-call variant word of the entry points: bit 0 selects the CUDA-core validation kernels, the
// B200MOE_GEMM_* bits restrict the tile shapes the tensor-core path may pick.  Nothing here is process state.
// `kind`: 0 = MX (a and b are element codes, K counts elements = bytes, or nibbles for e2m1 weights); 1 = dense
// bf16 operands (K counts bf16 elements; the copies address rows in bytes).
int run_gemm(int epi, const uint8_t* a, const uint8_t* b, GemmParams& p, int K, int impl, void* clock_probe,
             cudaStream_t st, int kind = 0) {
  B200MOE_REQUIRE((impl & ~(B200MOE_IMPL_SIMT | B200MOE_GEMM_TILE_N128 | B200MOE_GEMM_NO_PAIR | B200MOE_GEMM_FORCE_PAIR |
                            B200MOE_GEMM_NO_SPLIT | B200MOE_GEMM_NO_OVERLAP)) == 0,
                  B200MOE_ERR_INVALID, "unknown bits in the variant word 0x%x", impl);
  B200MOE_REQUIRE(clock_probe == nullptr || (reinterpret_cast<uintptr_t>(clock_probe) & 7) == 0, B200MOE_ERR_INVALID,
                  "the clock probe buffer must be 8-byte aligned");
  B200MOE_REQUIRE(p.B > 0 && p.B % 128 == 0, B200MOE_ERR_INVALID, "block size must be a multiple of 128, got %d", p.B);
  B200MOE_REQUIRE(K % 32 == 0 && K >= 32, B200MOE_ERR_INVALID, "contraction length must be a multiple of 32, got %d", K);
  B200MOE_REQUIRE(kind == 0 || !(impl & B200MOE_GEMM_TILE_N128), B200MOE_ERR_INVALID,
                  "the dense contraction has no 128-row weight tile");
  B200MOE_REQUIRE(p.n_blocks > 0 && p.E > 0 && p.E <= kMaxExperts, B200MOE_ERR_INVALID,
                  "need at least one block and between 1 and %d experts", kMaxExperts);
  B200MOE_REQUIRE(p.status != nullptr, B200MOE_ERR_INVALID, "status pointer must not be null");
  B200MOE_REQUIRE(p.w_format == B200MOE_W_E4M3 || p.w_format == B200MOE_W_E5M2 || p.w_format == B200MOE_W_E2M1,
                  B200MOE_ERR_INVALID, "unknown weight format %d", p.w_format);
  const bool nibbles = p.w_format == B200MOE_W_E2M1;
  B200MOE_REQUIRE(!nibbles || K % 128 == 0, B200MOE_ERR_INVALID,
                  "e2m1 weights need a contraction length that is a multiple of 128, got %d", K);
  p.m_tiles_total = p.n_blocks * (p.B / 128);
  p.clock_probe = static_cast<unsigned long long*>(clock_probe);
  const int Kb = kind == 1 ? 2 * K : K;  // row pitch the copies see, in element-code bytes
  p.k_blocks = (Kb + kBlockK - 1) / kBlockK;
  p.b_row_atoms = (p.n_total + 127) / 128;
  p.b_sf_expert_stride = static_cast<int64_t>(p.b_row_atoms) * p.k_blocks * 512;
  B200MOE_CUDA_OK(cudaMemsetAsync(p.status, 0, 4, st));
  if (impl & B200MOE_IMPL_SIMT) {
    const int64_t work = epi == 0 ? static_cast<int64_t>(p.m_tiles_total) * 128 * (p.I / 32)
                                  : static_cast<int64_t>(p.m_tiles_total) * 128 * p.H_out;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const int grid = static_cast<int>(ceil_div64(work, 128) < cap ? ceil_div64(work, 128) : cap);
    if (kind == 1) {
      const auto* ab = reinterpret_cast<const __nv_bfloat16*>(a);
      const auto* bb = reinterpret_cast<const __nv_bfloat16*>(b);
      if (epi == 0) simt_dense_gemm1_kernel<<<grid, 128, 0, st>>>(ab, bb, p, K);
      else simt_dense_gemm2_kernel<<<grid, 128, 0, st>>>(ab, bb, p, K);
    } else if (epi == 0) simt_gemm1_kernel<<<grid, 128, 0, st>>>(a, b, p, K);
    else simt_gemm2_kernel<<<grid, 128, 0, st>>>(a, b, p, K);
    B200MOE_LAUNCH_OK("simt_gemm_kernel");
    return B200MOE_OK;
  }
  B200MOE_REQUIRE(K % 16 == 0, B200MOE_ERR_INVALID, "TMA needs row pitches that are multiples of 16 bytes");
  const int bn = (impl & B200MOE_GEMM_TILE_N128) ? 128 : 256;
  const bool split_leftover = !(impl & B200MOE_GEMM_NO_SPLIT);
  const bool overlap_leftover = !(impl & B200MOE_GEMM_NO_OVERLAP);
  p.n_tiles = (p.n_total + bn - 1) / bn;
  // CTA pairs need two position tiles per weight tile: always there when a block holds an even number of 128-row
  // tiles; with odd blocks (B = 128) an expert's tiles are paired across its blocks, which pays once experts have
  // several tiles on average (prefill) and not for one short tile per expert (decode)
  const bool pair = !(impl & B200MOE_GEMM_NO_PAIR) && bn == 256 && (sm_count() % 2 == 0) &&
                    (p.B % 256 == 0 || (impl & B200MOE_GEMM_FORCE_PAIR) || p.m_tiles_total >= 4 * p.E);
  CUtensorMap ma[3], mb, mb128, msa, msb;  // activation boxes of 128, 64 and 32 rows; weight boxes: tile, 128 rows
  int rc = B200MOE_OK;
  for (int i = 0; i < 3 && rc == B200MOE_OK; ++i)
    rc = make_rows_map(&ma[i], a, Kb, static_cast<int64_t>(p.m_tiles_total) * 128, 0, kBlockM >> i);
  if (rc != B200MOE_OK) return rc;
  rc = make_rows_map(&mb, b, Kb, p.n_total, p.E, pair ? bn / 2 : bn, nibbles);
  // the copy reports the bytes it read from global memory: a 4-bit slab is 64 bytes per row there
  p.b_tx = static_cast<uint32_t>((pair ? bn / 2 : bn) * (nibbles ? kBlockK / 2 : kBlockK));
  if (rc != B200MOE_OK) return rc;
  rc = make_rows_map(&mb128, b, Kb, p.n_total, p.E, 128, nibbles);  // half tiles of the single-CTA launches
  if (rc != B200MOE_OK) return rc;
  if (kind == 0) {
    rc = make_atoms_map(&msa, p.a_sf, static_cast<int64_t>(p.m_tiles_total) * p.k_blocks);
    if (rc != B200MOE_OK) return rc;
    rc = make_atoms_map(&msb, p.b_sf, static_cast<int64_t>(p.E) * p.b_row_atoms * p.k_blocks);
    if (rc != B200MOE_OK) return rc;
  } else {
    msa = msb = ma[0];  // never dereferenced by the dense kernel
  }
  if (pair) {
    // Two launches: the CTA-pair kernel walks the pairs of live 128-row tiles, the single-CTA kernel the one
    // tile an expert with an odd number of live tiles has left over (a half-empty pair would pay for a full
    // 256-row MMA: with ~1000 rows per expert that was one tile in five).
    p.tile_filter = split_leftover ? 1 : 0;
    p.early_successor = (split_leftover && overlap_leftover) ? 1 : 0;
    if (kind == 1)
      rc = epi == 0 ? launch_tc<256, 6, 0, 2, 1>(ma, mb, mb128, msa, msb, p, st)
                    : launch_tc<256, 6, 1, 2, 1>(ma, mb, mb128, msa, msb, p, st);
    else
      rc = epi == 0 ? launch_tc<256, 6, 0, 2>(ma, mb, mb128, msa, msb, p, st) : launch_tc<256, 6, 1, 2>(ma, mb, mb128, msa, msb, p, st);
    if (rc != B200MOE_OK || !split_leftover) return rc;
    GemmParams p2 = p;
    p2.tile_filter = 2;
    p2.early_successor = 0;
    p2.wait_predecessor = overlap_leftover ? 1 : 0;
    p2.clock_probe = nullptr;
    p2.b_tx = static_cast<uint32_t>(bn * (nibbles ? kBlockK / 2 : kBlockK));
    CUtensorMap mb2;
    rc = make_rows_map(&mb2, b, Kb, p.n_total, p.E, bn, nibbles);
    if (rc != B200MOE_OK) return rc;
    const bool ov = overlap_leftover;
    if (kind == 1)
      return epi == 0 ? launch_tc<256, 4, 0, 1, 1>(ma, mb2, mb128, msa, msb, p2, st, ov)
                      : launch_tc<256, 4, 1, 1, 1>(ma, mb2, mb128, msa, msb, p2, st, ov);
    return epi == 0 ? launch_tc<256, 4, 0, 1>(ma, mb2, mb128, msa, msb, p2, st, ov)
                    : launch_tc<256, 4, 1, 1>(ma, mb2, mb128, msa, msb, p2, st, ov);
  }
  if (kind == 1)
    return epi == 0 ? launch_tc<256, 4, 0, 1, 1>(ma, mb, mb128, msa, msb, p, st)
                    : launch_tc<256, 4, 1, 1, 1>(ma, mb, mb128, msa, msb, p, st);
  if (bn == 256)
    return epi == 0 ? launch_tc<256, 4, 0, 1>(ma, mb, mb128, msa, msb, p, st) : launch_tc<256, 4, 1, 1>(ma, mb, mb128, msa, msb, p, st);
  return epi == 0 ? launch_tc<128, 6, 0, 1>(ma, mb, mb128, msa, msb, p, st) : launch_tc<128, 6, 1, 1>(ma, mb, mb128, msa, msb, p, st);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_grouped_gemm1_swiglu(const uint8_t* x_codes, const uint8_t* x_sf, const uint8_t* w1_dev,
                                            const uint8_t* w1_sf, int w_format, const float* bias_gu_dev,
                                            const int32_t* block_to_expert, const int32_t* conditions,
                                            const int32_t* tile_flags, int n_blocks, int B, int E, int H, int I,
                                            int act_fn, float gate_lo, float gate_hi, float up_lo, float up_hi,
                                            uint8_t* m_codes, uint8_t* m_sf, int32_t* status, int impl,
                                            void* clock_probe, b200moe_stream_t stream) {
  B200MOE_REQUIRE(x_codes && x_sf && w1_dev && w1_sf && block_to_expert && m_codes && m_sf, B200MOE_ERR_INVALID,
                  "grouped_gemm1: null pointer argument");
  B200MOE_REQUIRE(I % 32 == 0 && I > 0, B200MOE_ERR_INVALID, "grouped_gemm1: I must be a positive multiple of 32, got %d", I);
  B200MOE_REQUIRE(act_fn >= 0 && act_fn <= 3, B200MOE_ERR_INVALID, "grouped_gemm1: unknown activation %d", act_fn);
  B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(m_codes) & 31) == 0, B200MOE_ERR_INVALID,
                  "grouped_gemm1: m_codes must be 32-byte aligned (the epilogue stores 32 bytes at a time)");
  GemmParams p{};
  p.a_sf = x_sf;
  p.b_sf = w1_sf;
  p.w_format = w_format;
  p.block_to_expert = block_to_expert;
  p.conditions = conditions;
  p.tile_flags = tile_flags;
  p.n_blocks = n_blocks;
  p.B = B;
  p.E = E;
  p.n_total = 2 * I;
  p.bias = bias_gu_dev;
  p.act = act_fn;
  p.gate_lo = gate_lo;
  p.gate_hi = gate_hi;
  p.up_lo = up_lo;
  p.up_hi = up_hi;
  p.m_codes = m_codes;
  p.m_sf = m_sf;
  p.I = I;
  p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (I % 128 != 0)  // partially filled scale atoms along I must read as zero
    B200MOE_CUDA_OK(cudaMemsetAsync(m_sf, 0, b200moe_sf_bytes(static_cast<int64_t>(n_blocks) * B, I), st));
  return run_gemm(0, x_codes, w1_dev, p, H, impl, clock_probe, st);
}

namespace {
int gemm2_impl(const uint8_t* m_codes, const uint8_t* m_sf, const uint8_t* w2_dev, const uint8_t* w2_sf, int w_format,
               const float* bias_d, const int32_t* block_to_expert, const int32_t* conditions,
               const int32_t* tile_flags, const int32_t* token_position_to_id, int hidden_rows, int n_blocks, int B,
               int E, int H, int I, const void* affinities, int aff_dtype, int aff_per_row, void* y_pos_bf16,
               const int32_t* row_src, void* const* peer_out, int world, int64_t peer_rows, int32_t* status, int impl,
               void* clock_probe, b200moe_stream_t stream) {
  B200MOE_REQUIRE(m_codes && m_sf && w2_dev && w2_sf && block_to_expert && (y_pos_bf16 || row_src),
                  B200MOE_ERR_INVALID, "grouped_gemm2: null pointer argument");
  B200MOE_REQUIRE(H % 32 == 0 && H > 0, B200MOE_ERR_INVALID, "grouped_gemm2: H must be a positive multiple of 32, got %d", H);
  B200MOE_REQUIRE(aff_dtype == B200MOE_F32 || aff_dtype == B200MOE_BF16, B200MOE_ERR_INVALID,
                  "grouped_gemm2: affinities must be fp32 or bf16");
  GemmParams p{};
  p.a_sf = m_sf;
  p.b_sf = w2_sf;
  p.w_format = w_format;
  p.block_to_expert = block_to_expert;
  p.conditions = conditions;
  p.tile_flags = tile_flags;
  p.tpi = token_position_to_id;
  p.hidden_rows = hidden_rows;
  p.n_blocks = n_blocks;
  p.B = B;
  p.E = E;
  p.n_total = H;
  p.bias = bias_d;
  p.aff = affinities;
  p.aff_dtype = aff_dtype;
  p.aff_per_row = aff_per_row;
  p.y_pos = static_cast<__nv_bfloat16*>(y_pos_bf16);
  p.H_out = H;
  p.I = I;
  p.status = status;
  if (row_src != nullptr) {
    B200MOE_REQUIRE(peer_out != nullptr && world >= 1 && world <= 8 && token_position_to_id != nullptr,
                    B200MOE_ERR_INVALID, "grouped_gemm2: peer output needs 1..8 peer buffers and the row validity list");
    p.row_src = row_src;
    p.peer_rows = peer_rows;
    for (int i = 0; i < 8; ++i) p.peer_out[i] = i < world ? peer_out[i] : nullptr;
    for (int i = 0; i < world; ++i)
      B200MOE_REQUIRE(p.peer_out[i] != nullptr && (reinterpret_cast<uintptr_t>(p.peer_out[i]) & 31) == 0,
                      B200MOE_ERR_INVALID, "grouped_gemm2: peer buffer %d is null or not 32-byte aligned", i);
  } else {
    B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(y_pos_bf16) & 31) == 0, B200MOE_ERR_INVALID,
                    "grouped_gemm2: y_pos must be 32-byte aligned (the epilogue stores 32 bytes at a time)");
  }
  return run_gemm(1, m_codes, w2_dev, p, I, impl, clock_probe, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int b200moe_grouped_gemm2_scale(const uint8_t* m_codes, const uint8_t* m_sf, const uint8_t* w2_dev,
                                           const uint8_t* w2_sf, int w_format, const float* bias_d,
                                           const int32_t* block_to_expert, const int32_t* conditions,
                                           const int32_t* tile_flags, const int32_t* token_position_to_id,
                                           int hidden_rows, int n_blocks, int B, int E, int H, int I,
                                           const void* affinities, int aff_dtype, int aff_per_row, void* y_pos_bf16,
                                           int32_t* status, int impl, void* clock_probe,
                                           b200moe_stream_t stream) {
  return gemm2_impl(m_codes, m_sf, w2_dev, w2_sf, w_format, bias_d, block_to_expert, conditions, tile_flags,
                    token_position_to_id, hidden_rows, n_blocks, B, E, H, I, affinities, aff_dtype, aff_per_row,
                    y_pos_bf16, nullptr, nullptr, 0, 0, status, impl, clock_probe, stream);
}

extern "C" int b200moe_ep_gemm2_scale_return(const uint8_t* m_codes, const uint8_t* m_sf, const uint8_t* w2_dev,
                                             const uint8_t* w2_sf, int w_format, const float* bias_d,
                                             const int32_t* block_to_expert, const int32_t* conditions,
                                             const int32_t* tile_flags, const int32_t* row_valid, int64_t cap_rows,
                                             int n_blocks, int B, int E_local, int H, int I, const float* row_affinity,
                                             const int32_t* row_src, void* const* back_peers, int world,
                                             int64_t back_rows, int32_t* status, int impl, b200moe_stream_t stream) {
  B200MOE_REQUIRE(row_valid && row_src && back_peers, B200MOE_ERR_INVALID, "ep_gemm2_scale_return: null pointer argument");
  return gemm2_impl(m_codes, m_sf, w2_dev, w2_sf, w_format, bias_d, block_to_expert, conditions, tile_flags, row_valid,
                    static_cast<int>(cap_rows), n_blocks, B, E_local, H, I, row_affinity, B200MOE_F32, 1, nullptr,
                    row_src, back_peers, world, back_rows, status, impl, nullptr, stream);
}


// ---- dense (bf16) variants: the reference's non-MX expert kernels ------------------------------------------------
extern "C" int b200moe_dense_gemm1_swiglu(const void* x_bf16, const void* w1_bf16, const float* w1_col_scale,
                                          const float* bias_gu_dev, const int32_t* block_to_expert,
                                          const int32_t* conditions, const int32_t* tile_flags, int n_blocks, int B,
                                          int E, int H, int I, int act_fn, float gate_lo, float gate_hi, float up_lo,
                                          float up_hi, void* m_bf16, int32_t* status, int impl,
                                          b200moe_stream_t stream) {
  B200MOE_REQUIRE(x_bf16 && w1_bf16 && block_to_expert && m_bf16, B200MOE_ERR_INVALID,
                  "dense_gemm1: null pointer argument");
  B200MOE_REQUIRE(I % 32 == 0 && I > 0 && H % 32 == 0 && H > 0, B200MOE_ERR_INVALID,
                  "dense_gemm1: H and I must be positive multiples of 32 (H = %d, I = %d)", H, I);
  B200MOE_REQUIRE(act_fn >= 0 && act_fn <= 3, B200MOE_ERR_INVALID, "dense_gemm1: unknown activation %d", act_fn);
  B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(m_bf16) & 31) == 0, B200MOE_ERR_INVALID,
                  "dense_gemm1: the intermediate buffer must be 32-byte aligned");
  GemmParams p{};
  p.block_to_expert = block_to_expert;
  p.conditions = conditions;
  p.tile_flags = tile_flags;
  p.n_blocks = n_blocks;
  p.B = B;
  p.E = E;
  p.n_total = 2 * I;
  p.bias = bias_gu_dev;
  p.col_scale = w1_col_scale;
  p.act = act_fn;
  p.gate_lo = gate_lo;
  p.gate_hi = gate_hi;
  p.up_lo = up_lo;
  p.up_hi = up_hi;
  p.m_codes = static_cast<uint8_t*>(m_bf16);
  p.I = I;
  p.status = status;
  return run_gemm(0, static_cast<const uint8_t*>(x_bf16), static_cast<const uint8_t*>(w1_bf16), p, H, impl, nullptr,
                  static_cast<cudaStream_t>(stream), 1);
}

extern "C" int b200moe_dense_gemm2_scale(const void* m_bf16, const void* w2_bf16, const float* w2_col_scale,
                                         const float* bias_d, const int32_t* block_to_expert,
                                         const int32_t* conditions, const int32_t* tile_flags,
                                         const int32_t* token_position_to_id, int hidden_rows, int n_blocks, int B,
                                         int E, int H, int I, const void* affinities, int aff_dtype, int aff_per_row,
                                         void* y_pos_bf16, int32_t* status, int impl, b200moe_stream_t stream) {
  B200MOE_REQUIRE(m_bf16 && w2_bf16 && block_to_expert && y_pos_bf16, B200MOE_ERR_INVALID,
                  "dense_gemm2: null pointer argument");
  B200MOE_REQUIRE(H % 32 == 0 && H > 0 && I % 32 == 0 && I > 0, B200MOE_ERR_INVALID,
                  "dense_gemm2: H and I must be positive multiples of 32 (H = %d, I = %d)", H, I);
  B200MOE_REQUIRE(aff_dtype == B200MOE_F32 || aff_dtype == B200MOE_BF16, B200MOE_ERR_INVALID,
                  "dense_gemm2: affinities must be fp32 or bf16");
  B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(y_pos_bf16) & 31) == 0, B200MOE_ERR_INVALID,
                  "dense_gemm2: y_pos must be 32-byte aligned");
  GemmParams p{};
  p.block_to_expert = block_to_expert;
  p.conditions = conditions;
  p.tile_flags = tile_flags;
  p.tpi = token_position_to_id;
  p.hidden_rows = hidden_rows;
  p.n_blocks = n_blocks;
  p.B = B;
  p.E = E;
  p.n_total = H;
  p.bias = bias_d;
  p.col_scale = w2_col_scale;
  p.aff = affinities;
  p.aff_dtype = aff_dtype;
  p.aff_per_row = aff_per_row;
  p.y_pos = static_cast<__nv_bfloat16*>(y_pos_bf16);
  p.H_out = H;
  p.I = I;
  p.status = status;
  return run_gemm(1, static_cast<const uint8_t*>(m_bf16), static_cast<const uint8_t*>(w2_bf16), p, I, impl, nullptr,
                  static_cast<cudaStream_t>(stream), 1);
}
