// Grouped block-FP8 GEMM for sm_100a.
//
//   D[rows of group g, :] = sum over 128-wide K blocks kb of
//        a_scale[row, kb] * b_scale[g, n/128, kb] * (A_q[row, kb] . B_q[g, n, kb])
//
// A_q and B_q are E4M3; every 128-K block is multiplied on the tcgen05 tensor cores
// from a zeroed TMEM accumulator, drained by the epilogue warps and promoted into
// fp32 registers with the block's two scales, so FP8 accumulation never spans more
// than one scale block (the rule the reference's block GEMMs follow:
// src/mlops/kernels/block_fp8.py:217-223, kernels/quack_moe/block_fp8_gemm.py:1087-1136).
//
// One persistent CTA per SM, 12 warps:
//   warp 0      TMA producer (A tile 128x128 bytes, B tile BLOCK_N x 128 bytes per stage);
//               also draws the CTA's tiles from a global counter and publishes them to the
//               other roles (dynamic scheduling: see `tile_at` in the kernel)
//   warps 1, 3  UMMA issuers (one thread each), 4 x (128 x BLOCK_N x 32) per K block.  Even K
//               blocks (accumulator buffer 0) belong to warp 1, odd ones (buffer 1) to warp 3:
//               the two streams are independent, so while one thread is between K blocks
//               (commits, two barrier checks: a few hundred cycles) the tensor cores still
//               have the other thread's instructions queued
//   warp 2      TMEM allocation / release; in between it brings the scales of every K block (128
//               row scales, the tile's weight-block scales) from global memory into a ring in
//               shared memory and counts, with the operands, on the stage's `full` barrier
//   warp 3      first builds the tile table (group -> first M tile) in shared memory
//   warps 4-11  epilogue: tcgen05.ld of a K block's partial, scale, accumulate; at the
//               end of the K loop convert to bf16 and store the rows that belong to the
//               group (rows past the group's end were multiplied but are not written): 32 x 32
//               blocks through shared memory and TMA stores where all 32 rows belong to the
//               group, from registers otherwise.
// Two TMEM accumulator buffers let the tensor cores run K block k+1 while block k is
// being promoted.  No load is multicast; every wait is bounded.
#include "common.cuh"
#include "host_util.h"

#include <atomic>
#include <cstdlib>
#include <mutex>

namespace b200 {

constexpr int kMaxGroups = 1024;
constexpr int kBlockM = 128;
constexpr int kBlockK = 128;  // bytes == elements for E4M3
constexpr int kGemmThreads = 384;
constexpr int kScaleBatch = 4;  // K blocks of scales fetched ahead by the epilogue
constexpr uint32_t kAccBarrier = 1;  // hardware barriers 1, 2: accumulator buffer 0, 1 drained
constexpr uint32_t kAccBarrierThreads = (8 + 1) * 32;  // eight epilogue warps and the buffer's issuer

// Tile counters of the dynamic scheduler: [slot][0] next tile, [slot][1] CTAs that have finished.
// A slot belongs to ONE stream of one device (host-side table below): launches on a stream run
// one after the other, so no two launches that overlap on the GPU ever share a counter, and the
// last CTA of a launch leaves its slot zeroed for the next launch on that stream.  A launch that
// cannot be given a slot of its own (more than kSchedSlots streams seen on the device, a stream
// under capture -- a graph replay runs on whatever stream it is launched into --, or the
// per-thread default stream, one handle for many streams) gets sched_slot = -1 and strides over
// the tiles by CTA index instead.
constexpr int kSchedSlots = 64;
__device__ int g_tile_counter[kSchedSlots][2];

// In-kernel cycle counters (build with -DB200_GEMM_TRACE=1, see mlops_b200/build.py): CTA 0
// writes clock64() stamps of its roles for K blocks [kTraceFirst, kTraceFirst + kTraceIts) into
// a buffer handed over with b200moe_debug_set_gemm_trace: trace[slot][it - first][field].
//   slot 0 / 1  issuer of the even / odd K blocks: 0 loop top, 1 operands seen, 2 slab 0 free,
//               3 slab 0 issued, 4 slab 1 free, 5 slab 1 issued
//   slot 2 / 3  epilogue warp 4 (columns 0-127) / warp 8 (128-255): 0 waiting for the slab,
//               1 slab complete seen, 2 last TMEM load landed, 3 promoted and handed back; at the
//               first K block of a tile also 4 previous tile's store begins, 5 store issued,
//               6 next tile's number read, 7 next tile located
//   slot 4      producer: 0 waiting for the stage, 1 stage free (loads issued next)
#ifdef B200_GEMM_TRACE
constexpr int kTraceFirst = 64, kTraceIts = 64, kTraceFields = 8, kTraceSlots = 5;
#define B200_TRACE(slot, it, field)                                                                    \
  do {                                                                                                 \
    if (p.trace != nullptr && blockIdx.x == 0 && (int)(it) >= kTraceFirst && (int)(it) < kTraceFirst + kTraceIts) \
      p.trace[(((slot) * kTraceIts) + ((int)(it) - kTraceFirst)) * kTraceFields + (field)] = clock64();  \
  } while (0)
#else
#define B200_TRACE(slot, it, field) do {} while (0)
#endif

// Ablation builds (-DB200_GEMM_ABLATE=<bits>) take one part of the kernel's work out to show
// what the others cost; their results are wrong on purpose and the shipped library is built
// without them.  Bit 0: the epilogue hands an accumulator part back without reading it.
// Bit 1: it reads the part but skips the multiply-adds.  Bit 2: after the first fill of the
// stages the producer only signals them (no TMA traffic; the MMAs run on stale operands).
// Bit 3: the scales are taken as 1 instead of being fetched from global memory.
// -DB200_GEMM_FMA2=0 builds the scalar form of the promotion (one fmaf per element) for comparison.
#ifndef B200_GEMM_FMA2
#define B200_GEMM_FMA2 1
#endif
// (a0, a1) += s * (r0, r1), each element rounded like a scalar fmaf.
__device__ __forceinline__ void fma2(float& a0, float& a1, uint32_t r0, uint32_t r1, float s) {
  asm("{\n\t.reg .b64 a, r, sc;\n\t"
      "mov.b64 a, {%0, %1};\n\t"
      "mov.b64 r, {%2, %3};\n\t"
      "mov.b64 sc, {%4, %4};\n\t"
      "fma.rn.f32x2 a, r, sc, a;\n\t"
      "mov.b64 {%0, %1}, a;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "r"(r0), "r"(r1), "f"(s));
}
// -DB200_GEMM_VARIANT=<bits> builds alternatives of the per-K-block handshake that were measured
// against the shipped form (0) and lost or tied: bit 0 the issuers read the abort flag every
// eighth K block only, bit 1 / bit 2 the epilogue / the issuers wait with try_wait (sleeping)
// instead of polling, bit 3 an accumulator part is handed back before its last multiply-adds,
// bit 6 the epilogue warps fetch their scales from global memory themselves (no scale ring).
#ifndef B200_GEMM_VARIANT
#define B200_GEMM_VARIANT 0
#endif
#ifndef B200_GEMM_ABLATE
#define B200_GEMM_ABLATE 0
#endif

struct GemmFp8Params {
  const float* a_scale;
  long long as_row_stride, as_kb_stride;
  const float* b_scale;
  long long bs_group_stride, bs_n_stride, bs_k_stride;
  __nv_bfloat16* d;
  long long ldd;
  const __nv_bfloat16* addend;  // optional [rows, N] term added in fp32 before the rounding
  long long ldc;
  const int* offsets;
  int groups, N, K, rows_total;
  int weights;  // group g multiplies weight matrix g % weights
  // fused SwiGLU epilogue (EPI == 1): N = 2F, tiles pair 128 gate with 128 up columns
  uint8_t* act_q;
  long long ldq;
  float* act_scale;
  long long acts_row_stride, acts_kb_stride;
  float limit;
  int limited;
  // fused combine epilogue (EPI == 2): out_f32[row_token[r], :] += row_weight[r] * bf16(D[r, :])
  float* out_f32;
  long long ldo;
  const int* row_token;
  const float* row_weight;
  const int* row_map;  // optional: output row r is stored at d[row_map[r]] (NULL: in place)
  long long out_rows;  // rows of d (row_map) or of out_f32 (row_token): targets outside are skipped
  int sched_slot;      // slot of g_tile_counter, or -1: tiles by CTA index
  int wide_store;      // d's base and row pitch are multiples of 32 bytes: 32-byte stores per lane
  int tma_store;       // tmap_d describes d: full groups of 32 rows leave through TMA stores
  int* status;
#ifdef B200_GEMM_TRACE
  long long* trace;
#endif
#ifdef B200_WAIT_TEST
  int withhold_loads;  // test builds only: the producer issues no load, so every consumer's wait runs out
#endif
};

// PAIR: the two CTAs of a cluster share a 256-row x 256-column tile (tcgen05.mma.cta_group::2).
// CTA r holds rows [128 r, 128 r + 128) of A and, of each 128-column half of B, the 64 columns
// [64 r, 64 r + 64): every operand byte is written to shared memory once per pair (32 KB per
// CTA and K block instead of 48 KB), and a CTA's half of B is read once for both tensor cores.
template <int BLOCK_N, bool PAIR = false>
struct GemmCfg {
#ifdef B200_GEMM_STAGES
  static constexpr int kStages = B200_GEMM_STAGES;  // sensitivity builds only
#else
  static constexpr int kStages = (PAIR || BLOCK_N == 128) ? 6 : 4;
#endif
  static constexpr int kTileM = PAIR ? 2 * kBlockM : kBlockM;
  static constexpr int kABytes = kBlockM * kBlockK;
  static constexpr int kBBytes = (PAIR ? BLOCK_N / 2 : BLOCK_N) * kBlockK;
  static constexpr int kTmemCols = 2 * BLOCK_N;
  static constexpr int kTileBytes = kStages * (kABytes + kBBytes);
  static constexpr int kBarBytes = 512;
  static constexpr int kSchedBytes = (2 * (kMaxGroups + 1) * 4 + 15) / 16 * 16;
  // per-warp buffers of the epilogue's store: 32 rows x 64 bytes each, 1024-byte aligned (the
  // source of a TMA store in the 64-byte swizzle mode), plus the slack the alignment may cost
  // (one buffer per warp, or, where the stages leave room, one per 32-column block of the warp's
  // part of the tile, so that the blocks' bulk stores need not wait for one another)
  static constexpr int kFixedBytes = 1024 + kTileBytes + kBarBytes + kSchedBytes + 1024 + 8 * 136 * 4;
  static constexpr int kStoreBuffers = (232448 - kFixedBytes - 1024 >= 8 * 4 * 2048) ? 4 : 1;
  static constexpr int kStoreBytes = 8 * kStoreBuffers * 32 * 64 + 1024;
  // ring of the scales of eight K blocks (128 row scales, 4 block scales, padding), filled by warp 2
  static constexpr int kRingSlots = 8, kRingPitch = 136;
  static constexpr int kRingBytes = kRingSlots * kRingPitch * 4;
  static constexpr int kSmemBytes = 1024 + kTileBytes + kBarBytes + kSchedBytes + kStoreBytes + 1024 + kRingBytes;
};

struct TileCoord {
  int group, m0, rows_valid;
};

// m_tile_start[g] = number of M tiles in groups < g; offs[g] = first row of group g.
__device__ __forceinline__ TileCoord locate_m_tile(int mt, const int* m_tile_start, const int* offs,
                                                   int groups, int tile_m = kBlockM) {
  int lo = 0, hi = groups - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (m_tile_start[mid] <= mt) lo = mid; else hi = mid - 1;
  }
  // groups with zero tiles share a start with their successor; the search above lands on
  // the last group whose start <= mt, which is the one that owns the tile.
  TileCoord c;
  c.group = lo;
  c.m0 = offs[lo] + (mt - m_tile_start[lo]) * tile_m;
  c.rows_valid = min(tile_m, offs[lo + 1] - c.m0);
  return c;
}

// SPLIT (256-wide tile, plain or combining store): each K block is issued as two N=128
// halves into the two 128-column halves of its accumulator buffer, each with its own "full"
// mbarrier and its own hardware barrier for the release.  A half is drained by the four
// epilogue warps that own its columns, so the retire -> drain -> release -> reissue loop of
// one half runs beside the multiplication of the other three halves in flight.
//
// PAIR (with SPLIT): a cluster of two CTAs works on a 256 x 256 tile.  The leader CTA (cluster
// rank 0) issues every multiplication for both (tcgen05.mma.cta_group::2, M = 256, N = 128 per
// half); each CTA loads its own operands, drains its own 128 rows of the four accumulator
// slabs (2 buffers x 2 halves, all 512 TMEM columns) and stores them.  What crosses the pair:
// "my stage has landed" (a remote mbarrier arrival by warp 2 of each CTA), "this slab is
// drained" (remote arrivals by the epilogue warps on the leader's `tempty`), and the commits of
// the multiplications, which arrive on the barriers of both CTAs.  Four slabs in flight hide the
// retire -> drain -> release round trip behind the other three; half the B traffic per CTA
// leaves shared-memory bandwidth for it.  Tiles are assigned by pair index (no shared counter).
template <int BLOCK_N, bool B_MN_MAJOR, int EPI, bool SPLIT = false, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_d, const GemmFp8Params p) {
  using Cfg = GemmCfg<BLOCK_N, PAIR>;
  constexpr int kStages = Cfg::kStages;
  static_assert(!SPLIT || (BLOCK_N == 256 && EPI != 1), "the split issue is for the plain 256-wide tile");
  static_assert(!PAIR || (BLOCK_N == 256 && EPI == 0), "the pair form is the 256-wide tile with the plain store");
  constexpr int kHalves = SPLIT ? 2 : 1;  // separately released parts of an accumulator buffer
  // hardware barrier of (buffer, half); its participants: the warps that drain it and its issuer
  constexpr uint32_t kRelThreads = SPLIT ? (4 + 1) * 32 : kAccBarrierThreads;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * Cfg::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTileBytes);
  uint64_t* full = bars;                    // [kStages]
  uint64_t* empty = bars + kStages;         // [kStages]
  uint64_t* tfull = bars + 2 * kStages;     // [2 buffers][2 halves] (one per buffer unless SPLIT)
  // (an accumulator buffer, or half, is handed back to its issuer on a hardware barrier,
  // id 1 + buffer * halves + half, by the epilogue warps that drain it)
  uint64_t* drain = bars + 2 * kStages + 4;   // [2] one per issuer
  uint64_t* amax_bar = bars + 2 * kStages + 6;  // [4] row-quarter pairs of the fused SwiGLU epilogue
  uint64_t* sched_full = bars + 2 * kStages + 10;   // [4] ring of tile ids: slot published
  uint64_t* sched_empty = bars + 2 * kStages + 14;  // [4] ... and read by every consumer
  uint64_t* ready = bars + 2 * kStages + 18;        // [kStages] pair leader: both CTAs' stage landed
  uint64_t* tempty = bars + 3 * kStages + 18;       // [4] pair leader: slab drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 22);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* total_m_tiles_s = abort_flag + 1;
  int* sched_tile = total_m_tiles_s + 1;  // [4][4]: tile, its first row, rows that belong to the group, group
  int* m_tile_start = reinterpret_cast<int*>(smem + Cfg::kTileBytes + Cfg::kBarBytes);  // [groups+1]
  int* offs = m_tile_start + (kMaxGroups + 1);                                          // [groups+1]
  // Single-CTA form: warp 2 brings the two scales of every K block from global memory into a ring
  // in shared memory, one K block per operand stage, and counts on the stage's `full` barrier.
  // Fetched by the epilogue warps themselves, the loads held those warps up (a tenth of the
  // kernel's cycles) although they were issued four K blocks ahead.
  constexpr bool kScaleRing = !PAIR && (B200_GEMM_VARIANT & 64) == 0;
  float* scale_ring = reinterpret_cast<float*>(smem + Cfg::kTileBytes + Cfg::kBarBytes + Cfg::kSchedBytes +
                                               Cfg::kStoreBytes + 1024);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = p.groups;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int rank = PAIR ? (int)cluster_ctarank() : 0;  // 0: the CTA that issues the multiplications
  const bool leader = rank == 0;
  // EPI == 1: a tile is 128 gate columns and the 128 up columns that go with them
  const int half_n = p.N / 2;
  const int num_n_tiles = EPI == 1 ? half_n / 128 : (p.N + BLOCK_N - 1) / BLOCK_N;
  constexpr int kTileStep = EPI == 1 ? 128 : BLOCK_N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], kScaleRing ? 2 : 1);  // the operands (one arrival with their byte count) and the scales
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&tfull[i], 1);
    mbar_init(&drain[0], 1);
    mbar_init(&drain[1], 1);
    for (int i = 0; i < 4; ++i) mbar_init(&amax_bar[i], 64);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&sched_full[i], 1);
      // the readers of a tile id: eight epilogue warps, the issuer warps (two; none in the
      // pair's second CTA) and, in a pair, the warp that reports landed stages
      // (single-CTA form with the scale ring: warp 2 follows the tiles as well)
      mbar_init(&sched_empty[i], PAIR ? (leader ? 11 : 9) : (kScaleRing ? 11 : 10));
    }
    if constexpr (PAIR) {
      for (int s = 0; s < kStages; ++s) mbar_init(&ready[s], 2);  // one report per CTA
      // the epilogue warps of both CTAs that drain a slab (a half: four each; a buffer: eight)
      for (int i = 0; i < 4; ++i) mbar_init(&tempty[i], SPLIT ? 8 : 16);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  if (warp == 3) {
    // Tile table: exclusive scan of ceil(M_g / tile rows) over the groups.
    int running = 0;
    bool bad = false;
    for (int base = 0; base < groups; base += 32) {
      const int g = base + lane;
      int lo = 0, hi = 0;
      if (g < groups) {
        lo = p.offsets[g];
        hi = p.offsets[g + 1];
        if (lo < 0 || hi < lo || hi > p.rows_total) bad = true;
      }
      int tiles = (g < groups && !bad) ? (hi - lo + Cfg::kTileM - 1) / Cfg::kTileM : 0;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (g < groups) {
        m_tile_start[g] = running + incl - tiles;
        offs[g] = lo;
        if (g == groups - 1) offs[groups] = hi;
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
      m_tile_start[groups] = running;
      *total_m_tiles_s = bad ? 0 : running;
      if (bad) report_error(p.status, ERR_BAD_OFFSETS, 0, 0);
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before a remote arrival
  else __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = (*total_m_tiles_s) * num_n_tiles;
  // The 128 rows of M tile `mt` that this CTA loads, drains and stores.
  auto locate = [&](int mt) {
    TileCoord c = locate_m_tile(mt, m_tile_start, offs, groups, Cfg::kTileM);
    if constexpr (PAIR) {
      c.m0 += rank * kBlockM;
      c.rows_valid = max(0, min(kBlockM, c.rows_valid - rank * kBlockM));
    }
    return c;
  };

  // Tiles are handed out by a global counter, not by stride: a CTA that becomes resident late
  // (its SM was busy with another kernel, e.g. a collective) simply takes fewer tiles, and no
  // tile waits for a CTA that has not started.  The producer draws the numbers and publishes
  // them, one tile ahead, in a four-slot ring in shared memory; -1 ends the sequence.
  // `tile_at(i)`: the i-th tile of this CTA (warp-wide call; lane 0 waits); `done_with(i)`
  // lets the slot be reused.  -2: the wait gave up.
  // The producer locates a tile's rows (a binary search over the groups) once and publishes the
  // answer with the number, so the other roles do not repeat the search at every tile boundary.
  auto tile_at = [&](uint32_t i, TileCoord* where = nullptr) -> int {
    int t = -2, m0 = 0, rows_valid = 0, group = 0;
    if (lane == 0 && mbar_spin(&sched_full[i & 3], (i >> 2) & 1, abort_flag, p.status, 7)) {
      const volatile int* e = sched_tile + (i & 3) * 4;
      t = e[0];
      m0 = e[1];
      rows_valid = e[2];
      group = e[3];
    }
    if (where != nullptr) {
      where->m0 = __shfl_sync(0xffffffffu, m0, 0);
      where->rows_valid = __shfl_sync(0xffffffffu, rows_valid, 0);
      where->group = __shfl_sync(0xffffffffu, group, 0);
    }
    return __shfl_sync(0xffffffffu, t, 0);
  };
  auto done_with = [&](uint32_t i) {
    if (lane == 0) mbar_arrive(&sched_empty[i & 3]);
  };

  // The wide tile keeps 128 fp32 sums per epilogue thread: registers move from the
  // producer warpgroup (warps 0-3) to the two epilogue warpgroups.  Each role adjusts
  // its own limit at the top of its branch so the branches never merge in between.
#define B200_REG_DEC() do { if constexpr (BLOCK_N == 256) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); } while (0)
#define B200_REG_INC() do { if constexpr (BLOCK_N == 256) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); } while (0)

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    B200_REG_DEC();
    if (lane == 0) {
      uint32_t it = 0, published = 0;
      bool ok = true;
      uint32_t drawn = 0;
      auto draw = [&]() {
        int t;
        if constexpr (PAIR) t = (int)((blockIdx.x >> 1) + (drawn++) * (gridDim.x >> 1));  // by pair
        else t = p.sched_slot >= 0 ? atomicAdd(&g_tile_counter[p.sched_slot][0], 1)
                                   : (int)(blockIdx.x + (drawn++) * gridDim.x);
        return t < total_tiles ? t : -1;
      };
      auto publish = [&](int t) {
        const uint32_t slot = published & 3;
        if (!mbar_wait(&sched_empty[slot], ((published >> 2) & 1) ^ 1, abort_flag, p.status, 8)) return false;
        TileCoord where = {0, 0, 0};
        if (t >= 0) where = locate(t / num_n_tiles);
        sched_tile[slot * 4 + 0] = t;
        sched_tile[slot * 4 + 1] = where.m0;
        sched_tile[slot * 4 + 2] = where.rows_valid;
        sched_tile[slot * 4 + 3] = where.group;
        mbar_arrive(&sched_full[slot]);  // a release: the entry is visible to whoever sees the phase
        ++published;
        return true;
      };
      int t = draw();
      ok = publish(t);
      while (ok && t >= 0) {
        const int t_next = draw();
        if (!publish(t_next)) { ok = false; break; }  // the epilogue looks one tile ahead
        const int mt = t / num_n_tiles;
        const int n0 = (t - mt * num_n_tiles) * kTileStep;
        const TileCoord c = locate(mt);
        t = t_next;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          B200_TRACE(4, it, 0);
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          B200_TRACE(4, it, 1);
#ifdef B200_WAIT_TEST
          if (p.withhold_loads) continue;  // nothing is loaded and nothing arrives on full[s]
#endif
          if ((B200_GEMM_ABLATE & 4) && it >= (uint32_t)kStages) {
            mbar_arrive(&full[s]);
            continue;
          }
          mbar_arrive_expect_tx(&full[s], Cfg::kABytes + Cfg::kBBytes);
          tma_load_2d(sA + s * Cfg::kABytes, &tmap_a, &full[s], kb * kBlockK, c.m0);
          if constexpr (PAIR && SPLIT) {
            // this CTA's 64 columns of each 128-column half (two loads of 8 KB)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = n0 + h * 128 + rank * 64;
              if (!B_MN_MAJOR)
                tma_load_3d(sB + s * Cfg::kBBytes + h * (64 * kBlockK), &tmap_b, &full[s], kb * kBlockK, col,
                            c.group % p.weights);
              else
                tma_load_3d(sB + s * Cfg::kBBytes + h * (64 * kBlockK), &tmap_b, &full[s], col, kb * kBlockK,
                            c.group % p.weights);
            }
          } else if constexpr (PAIR) {
            // this CTA's 128 of the tile's 256 columns (one load of 16 KB)
            const int col = n0 + rank * 128;
            if (!B_MN_MAJOR)
              tma_load_3d(sB + s * Cfg::kBBytes, &tmap_b, &full[s], kb * kBlockK, col, c.group % p.weights);
            else
              tma_load_3d(sB + s * Cfg::kBBytes, &tmap_b, &full[s], col, kb * kBlockK, c.group % p.weights);
          } else if (EPI == 1) {
            tma_load_3d(sB + s * Cfg::kBBytes, &tmap_b, &full[s], kb * kBlockK, n0, c.group % p.weights);
            tma_load_3d(sB + s * Cfg::kBBytes + 128 * kBlockK, &tmap_b, &full[s], kb * kBlockK, half_n + n0,
                        c.group % p.weights);
          } else if (!B_MN_MAJOR) {
            tma_load_3d(sB + s * Cfg::kBBytes, &tmap_b, &full[s], kb * kBlockK, n0, c.group % p.weights);
          } else {
#pragma unroll
            for (int panel = 0; panel < BLOCK_N / 128; ++panel)
              tma_load_3d(sB + s * Cfg::kBBytes + panel * (128 * kBlockK), &tmap_b, &full[s],
                          n0 + panel * 128, kb * kBlockK, c.group % p.weights);
          }
        }
      }
      if (!ok) {
        // Unwinding: give the copies that were issued a bounded chance to land before
        // this CTA's shared memory is released.
#ifdef B200_WAIT_TEST
        const uint32_t issued = p.withhold_loads ? 0u : it;
#else
        const uint32_t issued = it;
#endif
        for (int s = 0; s < kStages; ++s) {
          if (issued <= (uint32_t)s) continue;
          const uint32_t last = ((issued - 1 - s) / kStages) * kStages + s;
          const uint32_t ph = (last / kStages) & 1;
          const long long start = clock64();
          while (!mbar_try(&full[s], ph) && clock64() - start < 20000000LL) {}
        }
      }
    }
  } else if (PAIR && warp == 2) {
    // ---- pair form: tell the leader CTA that this CTA's stage has landed.  The stage was
    // written by the async proxy (TMA), so the remote arrival needs no cluster-scope release.
    B200_REG_DEC();
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t tile_i = 0; ok; ++tile_i) {
      const int t = tile_at(tile_i);
      if (t == -2) ok = false;
      else done_with(tile_i);
      if (t < 0) break;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kStages;
        if (!mbar_wait_warp(&full[s], (it / kStages) & 1, abort_flag, p.status, 6)) { ok = false; break; }
        if (lane == 0) mbar_arrive_remote(&ready[s], 0);
      }
    }
  } else if (kScaleRing && warp == 2) {
    // ------------------------------ scale loader ------------------------------
    B200_REG_DEC();
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t tile_i = 0; ok; ++tile_i) {
      TileCoord c;
      const int t = tile_at(tile_i, &c);
      if (t == -2) ok = false;
      else done_with(tile_i);
      if (t < 0) break;
      const int n0 = (t % num_n_tiles) * kTileStep;
      // lane l holds the scales of rows l, l + 32, l + 64, l + 96 of the tile; lanes 0-3 also the
      // weight-block scales: [0], [1] of the columns of epilogue half 0, 1; [2], [3] of their up
      // columns (fused SwiGLU form).  Two K blocks per round of loads: this warp lives on 40
      // registers, and a round's latency is shorter than the operands' own.
      int row[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) row[i] = min(c.m0 + lane + 32 * i, p.rows_total - 1);
      const int h = lane & 1;
      const int col = (lane & 2) ? half_n + n0 + h * 64 : (EPI == 1 ? n0 + h * 64 : n0 + h * (BLOCK_N / 2));
      const float* b_ptr = p.b_scale + (long long)(c.group % p.weights) * p.bs_group_stride +
                           (long long)min(col / 128, (p.N - 1) / 128) * p.bs_n_stride;
      const bool has_b = lane < (EPI == 1 ? 4 : 2);
      for (int kb0 = 0; kb0 < num_kb && ok; kb0 += 2) {
        float va[2][4], vb[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int kk = min(kb0 + u, num_kb - 1);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            va[u][i] = p.a_scale[(long long)row[i] * p.as_row_stride + (long long)kk * p.as_kb_stride];
          vb[u] = has_b ? b_ptr[(long long)kk * p.bs_k_stride] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (kb0 + u >= num_kb) break;
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          // The stage's previous K block has been multiplied, so the K block that used this ring
          // slot (eight back) was promoted long ago: its accumulator had to be handed back before
          // a later one could be issued.
          if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag, p.status, 9)) { ok = false; break; }
          float* slot = scale_ring + (it % Cfg::kRingSlots) * Cfg::kRingPitch;
#pragma unroll
          for (int i = 0; i < 4; ++i) slot[lane + 32 * i] = va[u][i];
          if (has_b) slot[128 + lane] = vb[u];
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[s]);  // a release; the epilogue sees the slot through the issuer's commit
          ++it;
        }
      }
    }
  } else if ((warp == 1 || warp == 3) && (!PAIR || leader)) {
    // ------------------------------ UMMA issuers ------------------------------
    B200_REG_DEC();
    // The whole warp walks the loop (the hardware barrier counts warps); lane 0 issues.
    constexpr uint32_t idesc = make_idesc(0, 0, 0, B_MN_MAJOR ? 1 : 0, Cfg::kTileM, BLOCK_N / kHalves);
    const uint32_t mine = warp == 1 ? 0u : 1u;  // parity of the K blocks (and the buffer) of this warp
    uint32_t it = 0;  // K blocks since the kernel started: stage it % kStages, buffer it & 1
    bool ok = true;
    for (uint32_t tile_i = 0; ok; ++tile_i) {
      const int t = tile_at(tile_i);  // only whether there is another tile matters here
      if (t == -2) ok = false;         // the wait gave up
      else done_with(tile_i);
      if (t < 0) break;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((it & 1u) != mine) continue;
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        // the operands first: they have usually landed long ago, so this check is off the
        // path from the epilogue's release to the next multiplication
        if (lane == 0) B200_TRACE(mine, it, 0);
        if (!((B200_GEMM_VARIANT & 4) ? mbar_wait_warp(PAIR ? &ready[s] : &full[s], ph, abort_flag, p.status, 2)
                                      : mbar_spin_warp(PAIR ? &ready[s] : &full[s], ph, abort_flag, p.status, 2))) {
          ok = false;
          break;
        }
        if (lane == 0) B200_TRACE(mine, it, 1);
        // Everything the multiplications need is computed before the barrier: once the buffer
        // is free, the fewer instructions lane 0 still has to get through the scheduler (next
        // to epilogue warps that issue a multiply-add every cycle), the better.
        const uint64_t adesc = make_smem_desc(smem_u32(sA + s * Cfg::kABytes), 16, 1024);
        const uint32_t b_addr = smem_u32(sB + s * Cfg::kBBytes);
        // Pair form: this CTA's part of a half is 64 columns -- 64 K-major rows of 128 bytes, or
        // 128 MN-major K-rows of 64 bytes (64-byte swizzle, 8 rows = 512 bytes).
        constexpr bool kNarrowB = PAIR && SPLIT;  // 64 columns per CTA and multiplication
        const uint64_t bdesc = !B_MN_MAJOR ? make_smem_desc(b_addr, 16, 1024)
                               : kNarrowB  ? make_smem_desc(b_addr, 64 * kBlockK, 512, kLayoutSwizzle64)
                                           : make_smem_desc(b_addr, 128 * kBlockK, 1024);
        // K-major: 32 bytes further along the 128-byte swizzled row per MMA.
        // MN-major: 32 K-rows (of 128 bytes, or of 64 in a split pair) further.
        constexpr uint64_t kStepA = (uint64_t)(32 >> 4);
        constexpr uint64_t kStepB = (uint64_t)(B_MN_MAJOR ? ((32 * (kNarrowB ? 64 : 128)) >> 4) : (32 >> 4));
        // one half further: 128 columns of B (16 KB), of which a pair's CTA holds 64 (8 KB)
        constexpr uint64_t kHalfB = (uint64_t)(((kNarrowB ? 64 : 128) * kBlockK) >> 4);
        const uint32_t empty_bar = smem_u32(&empty[s]);
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
          const uint64_t bdesc_h = bdesc + (uint64_t)h * kHalfB;
          const uint32_t d_tmem = tmem_base + mine * BLOCK_N + h * 128;
          const uint32_t tfull_bar = smem_u32(&tfull[mine * kHalves + h]);
          if (it >= 2) {
            // this part of the buffer holds an earlier K block: its readers hand it back here.
            if constexpr (PAIR) {
              // ... the epilogue warps of both CTAs, by remote arrivals on the leader's barrier
              if (!mbar_spin_warp(&tempty[mine * kHalves + h], ((it >> 1) - 1) & 1, abort_flag, p.status, 3)) {
                ok = false;
                break;
              }
            } else {
              // An epilogue warp that unwinds arrives once more, so this cannot wait forever.
              named_sync(kAccBarrier + mine * kHalves + h, kRelThreads);
            }
          }
          if (lane == 0) {
            B200_TRACE(mine, it, 2 + 2 * h);
            tc_fence_after_sync();
            if constexpr (PAIR) {
              umma_f8_pair(d_tmem, adesc, bdesc_h, idesc, 0u);
              umma_f8_pair(d_tmem, adesc + kStepA, bdesc_h + kStepB, idesc, 1u);
              umma_f8_pair(d_tmem, adesc + 2 * kStepA, bdesc_h + 2 * kStepB, idesc, 1u);
              umma_f8_pair(d_tmem, adesc + 3 * kStepA, bdesc_h + 3 * kStepB, idesc, 1u);
              umma_commit_pair(&tfull[mine * kHalves + h], 3);  // the epilogues of both CTAs
              if (h == kHalves - 1) umma_commit_pair(&empty[s], 3);  // ... and both producers
            } else {
              umma_f8(d_tmem, adesc, bdesc_h, idesc, 0u);
              umma_f8(d_tmem, adesc + kStepA, bdesc_h + kStepB, idesc, 1u);
              umma_f8(d_tmem, adesc + 2 * kStepA, bdesc_h + 2 * kStepB, idesc, 1u);
              umma_f8(d_tmem, adesc + 3 * kStepA, bdesc_h + 3 * kStepB, idesc, 1u);
              umma_commit_addr(tfull_bar);
              if (h == kHalves - 1) umma_commit_addr(empty_bar);
            }
            B200_TRACE(mine, it, 3 + 2 * h);
          }
        }
        if (!ok) break;
        // one lane reads the flag so that the warp leaves the loop together (a warp that split
        // here would come back to the hardware barrier with lanes missing)
        if (!(B200_GEMM_VARIANT & 1) || (it & 15u) == mine) {
          int aborted = lane == 0 ? *abort_flag : 0;
          aborted = __shfl_sync(0xffffffffu, aborted, 0);
          if (aborted) { ok = false; break; }
        }
      }
    }
    if (!ok && lane == 0) {
      if constexpr (PAIR) umma_commit_pair(&drain[mine], 1);
      else umma_commit(&drain[mine]);
      const long long start = clock64();
      while (!mbar_try(&drain[mine], 0) && clock64() - start < 20000000LL) {}
    }
  } else if (warp >= 4) {
    // ------------------------------- epilogue --------------------------------
    B200_REG_INC();
    constexpr int kCols = BLOCK_N / 2;  // columns owned by one thread
    constexpr int kChunks = kCols / 32;
    // A row of a warp's buffer is 64 bytes; its four 16-byte pieces are stored swizzled
    // (piece ^ ((row >> 1) & 3)): conflict-free for a lane-per-row write and for the 8 rows x 4
    // pieces read, and the layout a TMA store with the 64-byte swizzle expects.
    constexpr int kStageRowBytes = 64;
    constexpr int kStageWarpBytes = 32 * kStageRowBytes;
    auto piece_at = [](int row, int piece) { return row * kStageRowBytes + ((piece ^ ((row >> 1) & 3)) << 4); };
    uint8_t* stage_base = smem + Cfg::kTileBytes + Cfg::kBarBytes + Cfg::kSchedBytes;
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;   // which half of the tile's columns
    const int row_in_tile = q * 32 + lane;
    float acc[kCols];
    uint32_t ab = 0;
    uint32_t amax_phase = 0;
    bool ok = true;
    float* amax_s = reinterpret_cast<float*>(stage_base + Cfg::kStoreBytes);  // [2][128]

    // Everything the epilogue needs to know about one tile.
    struct EpiTile {
      int rows_valid, grow, col0, col1;  // col1: first up column of this thread (EPI == 1)
      const float* as_ptr;
      const float* bs_ptr;
      const float* bs_ptr_up;
    };
    auto describe = [&](int t, const TileCoord& c) {
      EpiTile e;
      const int n0 = (t % num_n_tiles) * kTileStep;
      e.rows_valid = c.rows_valid;
      e.grow = c.m0 + row_in_tile;
      e.col0 = EPI == 1 ? n0 + half * 64 : n0 + half * kCols;
      e.col1 = half_n + e.col0;
      e.as_ptr = p.a_scale + (long long)min(e.grow, p.rows_total - 1) * p.as_row_stride;
      e.bs_ptr = p.b_scale + (long long)(c.group % p.weights) * p.bs_group_stride +
                 (long long)min(e.col0 / 128, (p.N - 1) / 128) * p.bs_n_stride;
      e.bs_ptr_up = p.b_scale + (long long)(c.group % p.weights) * p.bs_group_stride +
                    (long long)min(e.col1 / 128, (p.N - 1) / 128) * p.bs_n_stride;
      return e;
    };
    // The two scales of a K block come from global memory.  They are fetched one batch of
    // kScaleBatch K blocks ahead -- across the tile boundary too -- so their latency never
    // sits between two K blocks.
    float sa_cur[kScaleBatch], sb_cur[kScaleBatch], sa_nxt[kScaleBatch], sb_nxt[kScaleBatch];
    float su_cur[EPI == 1 ? kScaleBatch : 1], su_nxt[EPI == 1 ? kScaleBatch : 1];  // up-column block scales
    auto fetch = [&](const EpiTile& e, int kb0, float (&sa)[kScaleBatch], float (&sb)[kScaleBatch],
                     float (&su)[EPI == 1 ? kScaleBatch : 1]) {
#pragma unroll
      for (int u = 0; u < kScaleBatch; ++u) {
        if constexpr ((B200_GEMM_ABLATE & 8) != 0) {  // no scale traffic
          sa[u] = 1.f;
          sb[u] = 1.f;
          if constexpr (EPI == 1) su[u] = 1.f;
          continue;
        }
        const int kk = min(kb0 + u, num_kb - 1);
        sa[u] = e.as_ptr[(long long)kk * p.as_kb_stride];
        sb[u] = e.bs_ptr[(long long)kk * p.bs_k_stride];
        if constexpr (EPI == 1) su[u] = e.bs_ptr_up[(long long)kk * p.bs_k_stride];
      }
    };
    EpiTile cur_tile, nxt_tile;
    TileCoord where;
    int t_cur = tile_at(0, &where);
    if (t_cur == -2) ok = false;
    if (t_cur >= 0) {
      cur_tile = describe(t_cur, where);
      if constexpr (!kScaleRing) fetch(cur_tile, 0, sa_cur, sb_cur, su_cur);
    }
    for (uint32_t tile_i = 0; t_cur >= 0 && ok; ++tile_i) {
      if (lane == 0 && q == 0) B200_TRACE(2 + half, ab, 5);
      const int t_nxt = tile_at(tile_i + 1, &where);  // published together with the current one
      if (t_nxt == -2) { ok = false; break; }
      if (lane == 0 && q == 0) B200_TRACE(2 + half, ab, 6);
      const bool has_next = t_nxt >= 0;
      if (has_next) nxt_tile = describe(t_nxt, where);
      done_with(tile_i);
      if (lane == 0 && q == 0) B200_TRACE(2 + half, ab, 7);
      t_cur = t_nxt;
      const EpiTile c = cur_tile;
      const int grow = c.grow;
      const int col0 = c.col0;
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
      for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kScaleBatch) {
        if constexpr (!kScaleRing) {
          if (kb0 + kScaleBatch < num_kb) fetch(c, kb0 + kScaleBatch, sa_nxt, sb_nxt, su_nxt);
          else if (has_next) fetch(nxt_tile, 0, sa_nxt, sb_nxt, su_nxt);
        }
#pragma unroll
        for (int u = 0; u < kScaleBatch; ++u) {
          if (kb0 + u >= num_kb) break;
          float s = 0.f, s_up = 0.f;
          if constexpr (!kScaleRing) {
            s = sa_cur[u] * sb_cur[u];
            s_up = EPI == 1 ? sa_cur[u] * su_cur[u] : s;
          }
          const int buf = ab & 1;
          const uint32_t aph = (ab >> 1) & 1;
          ++ab;
          const int part = SPLIT ? buf * 2 + half : buf;  // what this warp waits for and hands back
          if (lane == 0 && q == 0) B200_TRACE(2 + half, ab - 1, 0);
          if (!((B200_GEMM_VARIANT & 2) ? mbar_wait_warp(&tfull[part], aph, abort_flag, p.status, 4)
                                        : mbar_spin_warp(&tfull[part], aph, abort_flag, p.status, 4))) {
            ok = false;
            break;
          }
          if (lane == 0 && q == 0) B200_TRACE(2 + half, ab - 1, 1);
          if constexpr (kScaleRing) {
            // written before the stage's `full` barrier completed, which the issuer saw before it
            // issued what this warp has just seen complete
            const float* slot = scale_ring + ((ab - 1) % Cfg::kRingSlots) * Cfg::kRingPitch;
            const float sa = slot[row_in_tile];
            s = sa * slot[128 + half];
            s_up = EPI == 1 ? sa * slot[130 + half] : s;
          }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BLOCK_N +
                                 (EPI == 1 ? half * 64 : half * kCols);
          // EPI == 1: chunks 0,1 are this thread's 64 gate columns, chunks 2,3 its 64 up columns.
          // Two tcgen05.ld are kept in flight.
          auto tcol = [&](int cc) { return EPI == 1 ? (cc & 1) * 32 + (cc >> 1) * 128 : cc * 32; };
          auto promote = [&](const uint32_t (&r)[32], int cc) {
            const float sc = (EPI == 1 && cc >= 2) ? s_up : s;
            if constexpr ((B200_GEMM_ABLATE & 2) != 0) {
              acc[cc * 32] += sc * __uint_as_float(r[0]);
              return;
            }
#if B200_GEMM_FMA2
            // two multiply-adds per instruction (fma.rn.f32x2): same roundings, half the issue slots
#pragma unroll
            for (int j = 0; j < 32; j += 2) fma2(acc[cc * 32 + j], acc[cc * 32 + j + 1], r[j], r[j + 1], sc);
#else
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[cc * 32 + j] = fmaf(sc, __uint_as_float(r[j]), acc[cc * 32 + j]);
#endif
          };
          auto release = [&]() {
            tc_fence_before_sync();
            __syncwarp();
            if constexpr (PAIR) {
              if (lane == 0) mbar_arrive_remote(&tempty[part], 0);  // the leader issues for both CTAs
            } else {
              named_arrive(kAccBarrier + part, kRelThreads);
            }
          };
          if constexpr ((B200_GEMM_ABLATE & 1) != 0) {
            acc[0] += s + s_up;
            release();
            continue;
          }
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(taddr + tcol(0), ra);
          tmem_ld_32x32(taddr + tcol(1), rb);
          tmem_ld_wait();
          if constexpr (kChunks == 2) {
            release();
            promote(ra, 0);
            promote(rb, 1);
          } else {
            static_assert(kChunks == 4, "tile widths are 128 or 256");
            promote(ra, 0);
            tmem_ld_32x32(taddr + tcol(2), ra);
            promote(rb, 1);
            tmem_ld_32x32(taddr + tcol(3), rb);
            tmem_ld_wait();
            if (lane == 0 && q == 0) B200_TRACE(2 + half, ab - 1, 2);
            // The buffer is handed back only after the last multiply-adds: released earlier,
            // the 64 FMAs that follow (one per cycle, from both epilogue warps of a
            // sub-partition) keep the issuer warp from being scheduled, and the next
            // multiplication starts later than if the release had simply waited for them.
            if constexpr ((B200_GEMM_VARIANT & 8) != 0) {
              release();
              promote(ra, 2);
              promote(rb, 3);
            } else {
              promote(ra, 2);
              promote(rb, 3);
              release();
            }
            if (lane == 0 && q == 0) B200_TRACE(2 + half, ab - 1, 3);
          }
        }
        if constexpr (!kScaleRing) {
#pragma unroll
          for (int u = 0; u < kScaleBatch; ++u) {
            sa_cur[u] = sa_nxt[u];
            sb_cur[u] = sb_nxt[u];
            if constexpr (EPI == 1) su_cur[u] = su_nxt[u];
          }
        }
      }
      cur_tile = nxt_tile;
      if (!ok) break;
      if (lane == 0 && q == 0) B200_TRACE(2 + half, ab, 4);
      // Store: the warp holds 32 rows x kCols columns, one row per lane.  Written directly, a
      // store instruction would touch 32 different rows with 16 bytes each; instead each 32-column
      // slab goes through a small per-warp shared-memory buffer and leaves as 8 rows x 64
      // contiguous bytes per instruction (whole 32-byte sectors).
      {
        uint8_t* stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(stage_base) + 1023) & ~uintptr_t(1023)) +
                         (warp - 4) * (Cfg::kStoreBuffers * kStageWarpBytes);
        bool drained = false;  // several buffers: one wait per tile covers the previous tile's stores
        // a bulk store of this warp may still be reading the buffer; lane 0 issued them all
        auto buffer_free = [&]() {
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
        };
        const int rows_here = c.rows_valid - q * 32;  // rows of this warp that belong to the group
        // where this lane's row goes: in place, or wherever the caller's map sends it (rows
        // that arrived as [source rank][expert] and were multiplied in expert order go back)
        int out_row = (p.row_map != nullptr && lane < rows_here) ? p.row_map[grow] : grow;
        if (p.row_map != nullptr && lane < rows_here && (out_row < 0 || out_row >= p.out_rows)) {
          report_error(p.status, ERR_BAD_OFFSETS, 11, grow);  // a map entry outside d: row not stored
          out_row = -1;
        }
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
          if (p.addend != nullptr && lane < rows_here) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + cc * 32 + j + 8 <= p.N) {
                const uint4 raw = *reinterpret_cast<const uint4*>(p.addend + (long long)grow * p.ldc + col0 +
                                                                  cc * 32 + j);
                const __nv_bfloat162* cv = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 f = __bfloat1622float2(cv[u]);
                  acc[cc * 32 + j + 2 * u] += f.x;
                  acc[cc * 32 + j + 2 * u + 1] += f.y;
                }
              }
            }
          }
          if constexpr (EPI == 2) {
            // Combine fused into the store: the row, rounded to bf16 as the stored expert
            // output would be, times its route weight, is added to the token's fp32 row
            // with 16-byte atomics (4 rows x 64 contiguous bytes per instruction after the
            // same shared-memory transpose as the plain store).  The K experts of a token
            // arrive in no fixed order, so the sum is not bitwise repeatable: the plain
            // store plus `combine_kernel` is.
            int tok = lane < rows_here ? p.row_token[grow] : 0;
            const float wgt = lane < rows_here ? p.row_weight[grow] : 0.f;
            if (tok < 0 || tok >= p.out_rows) {
              report_error(p.status, ERR_BAD_OFFSETS, 12, grow);  // no such token: row not added
              tok = -1;
            }
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              buffer_free();
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                float4 v;
                v.x = wgt * __bfloat162float(__float2bfloat16_rn(acc[cc * 32 + sub * 16 + j + 0]));
                v.y = wgt * __bfloat162float(__float2bfloat16_rn(acc[cc * 32 + sub * 16 + j + 1]));
                v.z = wgt * __bfloat162float(__float2bfloat16_rn(acc[cc * 32 + sub * 16 + j + 2]));
                v.w = wgt * __bfloat162float(__float2bfloat16_rn(acc[cc * 32 + sub * 16 + j + 3]));
                *reinterpret_cast<float4*>(stage + piece_at(lane, j >> 2)) = v;
              }
              __syncwarp();
              const int piece = lane & 3;  // 16-byte piece of the 64-byte row slab
              const int col = col0 + cc * 32 + sub * 16 + piece * 4;
#pragma unroll
              for (int pass = 0; pass < 4; ++pass) {
                const int r = pass * 8 + (lane >> 2);
                const int tok_r = __shfl_sync(0xffffffffu, tok, r);
                if (r < rows_here && tok_r >= 0 && col + 4 <= p.N) {
                  const float4 v = *reinterpret_cast<const float4*>(stage + piece_at(r, piece));
                  atomicAdd(reinterpret_cast<float4*>(p.out_f32 + (long long)tok_r * p.ldo + col), v);
                }
              }
            }
            continue;
          }
          const int chunk_col0 = EPI == 1 ? ((cc >> 1) ? c.col1 : c.col0) + (cc & 1) * 32 : col0 + cc * 32;
          if (p.tma_store && rows_here >= 32 && chunk_col0 + 32 <= p.N) {
            // All 32 rows of the warp belong to the group and lie one after the other in d: the
            // 32 x 32 block goes to a 2 KB buffer (rows of 64 bytes, 16-byte pieces swizzled as the
            // tensor map's 64-byte mode expects: conflict-free writes) and leaves as ONE bulk
            // store.  Written from registers, the tile's 2048 sector-sized stores per CTA kept the
            // SM's memory pipeline busy for thousands of cycles, in which the issuers' own
            // instructions (multiplications, barrier checks) queued behind them.  A bulk store
            // needs some 700 cycles to read its buffer: with one buffer per warp the four blocks
            // wait for one another, with four they do not.
            uint8_t* out = stage;
            if constexpr (Cfg::kStoreBuffers > 1) {
              out = stage + (cc % Cfg::kStoreBuffers) * kStageWarpBytes;
              if (!drained) buffer_free();
              drained = true;
            } else {
              buffer_free();  // the previous block has left the buffer
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(acc[cc * 32 + j * 8 + 0], acc[cc * 32 + j * 8 + 1]);
              v.y = pack_bf16x2(acc[cc * 32 + j * 8 + 2], acc[cc * 32 + j * 8 + 3]);
              v.z = pack_bf16x2(acc[cc * 32 + j * 8 + 4], acc[cc * 32 + j * 8 + 5]);
              v.w = pack_bf16x2(acc[cc * 32 + j * 8 + 6], acc[cc * 32 + j * 8 + 7]);
              *reinterpret_cast<uint4*>(out + piece_at(lane, j)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_d, out, chunk_col0, c.grow - lane);
              bulk_commit_group();
            }
            continue;
          }
          if (p.wide_store && chunk_col0 + 32 <= p.N) {
            // 32 bytes per lane and instruction straight from the registers: whole sectors of the
            // lane's own row, no trip through shared memory (the store phase of a tile holds up the
            // next tile's accumulators, so its length counts: 16 K blocks per tile in the down
            // projection)
            if (lane < rows_here && out_row >= 0) {
              __nv_bfloat16* drow = p.d + (long long)out_row * p.ldd + chunk_col0;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(drow + h * 16),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 0], acc[cc * 32 + h * 16 + 1])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 2], acc[cc * 32 + h * 16 + 3])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 4], acc[cc * 32 + h * 16 + 5])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 6], acc[cc * 32 + h * 16 + 7])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 8], acc[cc * 32 + h * 16 + 9])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 10], acc[cc * 32 + h * 16 + 11])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 12], acc[cc * 32 + h * 16 + 13])),
                             "r"(pack_bf16x2(acc[cc * 32 + h * 16 + 14], acc[cc * 32 + h * 16 + 15]))
                             : "memory");
              }
            }
            continue;
          }
          buffer_free();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            v.x = pack_bf16x2(acc[cc * 32 + j + 0], acc[cc * 32 + j + 1]);
            v.y = pack_bf16x2(acc[cc * 32 + j + 2], acc[cc * 32 + j + 3]);
            v.z = pack_bf16x2(acc[cc * 32 + j + 4], acc[cc * 32 + j + 5]);
            v.w = pack_bf16x2(acc[cc * 32 + j + 6], acc[cc * 32 + j + 7]);
            *reinterpret_cast<uint4*>(stage + piece_at(lane, j >> 3)) = v;
          }
          __syncwarp();
          const int piece = lane & 3;          // 16-byte piece of the 64-byte row slab
          const int chunk_col = EPI == 1 ? ((cc >> 1) ? c.col1 : c.col0) + (cc & 1) * 32 : col0 + cc * 32;
          const int col = chunk_col + piece * 8;
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            const int r = pass * 8 + (lane >> 2);
            const int dst_row = __shfl_sync(0xffffffffu, out_row, r);
            if (r < rows_here && dst_row >= 0 && col + 8 <= p.N) {
              const uint4 v = *reinterpret_cast<const uint4*>(stage + piece_at(r, piece));
              *reinterpret_cast<uint4*>(p.d + (long long)dst_row * p.ldd + col) = v;
            }
          }
        }
        if constexpr (EPI == 1) {
          // act = silu(gate) * up from the bf16 values just stored (what a separate pass over
          // h13 would read), one E4M3 scale per row and 128 columns: the other half of the
          // block lives in the partner warp (same rows, other 64 columns), so the two exchange
          // their maxima through shared memory with a bounded mbarrier wait.
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            float gi = __bfloat162float(__float2bfloat16_rn(acc[j]));
            float ui = __bfloat162float(__float2bfloat16_rn(acc[64 + j]));
            if (p.limited) {
              gi = fminf(gi, p.limit);
              ui = fminf(fmaxf(ui, -p.limit), p.limit);
            }
            const float sig = __frcp_rn(1.0f + expf(-gi));
            acc[j] = gi * sig * ui;
            amax = fmaxf(amax, fabsf(acc[j]));
          }
          amax_s[half * 128 + row_in_tile] = amax;
          mbar_arrive(&amax_bar[q]);
          if (!__all_sync(0xffffffffu, mbar_wait(&amax_bar[q], amax_phase, abort_flag, p.status, 5))) {
            ok = false;
            break;
          }
          amax_phase ^= 1;
          amax = fmaxf(amax, amax_s[(half ^ 1) * 128 + row_in_tile]);
          const float scale = fmaxf(amax * kInv448, 1e-12f);
          if (lane < rows_here) {
            uint8_t* arow = p.act_q + (long long)grow * p.ldq + c.col0;
#pragma unroll
            for (int j = 0; j < 64; j += 16) {
              float v0[8], v1[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                v0[i] = acc[j + i];
                v1[i] = acc[j + 8 + i];
              }
              const uint2 lo8 = quantize8(v0, scale), hi8 = quantize8(v1, scale);
              *reinterpret_cast<uint4*>(arow + j) = make_uint4(lo8.x, lo8.y, hi8.x, hi8.y);
            }
            if (half == 0)
              p.act_scale[(long long)grow * p.acts_row_stride + (long long)(c.col0 >> 7) * p.acts_kb_stride] = scale;
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();  // the buffers' last bulk stores, before shared memory is given up
    if (!ok) {
      // Unwinding: an issuer may be waiting on a hardware barrier for this warp.  (In the pair
      // form the issuer's wait is an mbarrier wait with its own limit.)
      if constexpr (!PAIR) {
        named_arrive(kAccBarrier + (SPLIT ? half : 0), kRelThreads);
        named_arrive(kAccBarrier + (SPLIT ? 2 + half : 1), kRelThreads);
      }
    }
  }

  else {
    B200_REG_DEC();
  }
#undef B200_REG_DEC
#undef B200_REG_INC

  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();  // the peer may still be arriving on, or reading from, this CTA
  else __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  // The thread that drew this CTA's tiles reports the CTA finished; the last one in the grid
  // leaves the slot zeroed for a later launch.
  if (!PAIR && threadIdx.x == 0 && p.sched_slot >= 0) {
    const int finished = atomicAdd(&g_tile_counter[p.sched_slot][1], 1);
    if (finished == (int)gridDim.x - 1) {
      g_tile_counter[p.sched_slot][0] = 0;
      g_tile_counter[p.sched_slot][1] = 0;
    }
  }
}

// The scheduler slot of (current device, stream), or -1 when the launch must not draw its
// tiles from a shared counter (see g_tile_counter).
static int sched_slot_of(cudaStream_t stream) {
  if (stream == cudaStreamPerThread) return -1;
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return -1;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  static std::mutex lock;
  static cudaStream_t table[64][kSchedSlots];
  static int used[64];
  std::lock_guard<std::mutex> guard(lock);
  // the legacy default stream has two spellings; both are slot 0's key
  const cudaStream_t key = (stream == nullptr) ? cudaStreamLegacy : stream;
  for (int i = 0; i < used[dev]; ++i)
    if (table[dev][i] == key) return i;
  if (used[dev] == kSchedSlots) return -1;
  table[dev][used[dev]] = key;
  return used[dev]++;
}

// The pair form: clusters of two CTAs, one 256 x 256 tile per pair at a time.
template <bool B_MN, bool SPLIT>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmFp8Params& p, cudaStream_t stream) {
  using Cfg = GemmCfg<256, true>;
  auto kern = grouped_gemm_fp8_kernel<256, B_MN, 0, SPLIT, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
    return B200MOE_ERR_LAUNCH;
  const long long m_tiles_bound = (p.rows_total + Cfg::kTileM - 1) / Cfg::kTileM + p.groups;
  const long long tiles = m_tiles_bound * ((p.N + 255) / 256);
  long long pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  GemmFp8Params q = p;
  q.sched_slot = -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, td, q) != cudaSuccess) return B200MOE_ERR_LAUNCH;
  return launch_status();
}

template <int BLOCK_N, bool B_MN, int EPI = 0, bool SPLIT = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                       const GemmFp8Params& p, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N>;
  auto kern = grouped_gemm_fp8_kernel<BLOCK_N, B_MN, EPI, SPLIT>;
  // Function attributes are per device; setting one is a cheap host-side call.
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
    return B200MOE_ERR_LAUNCH;
  const long long m_tiles_bound = (p.rows_total + kBlockM - 1) / kBlockM + p.groups;
  const long long n_tiles = EPI == 1 ? p.N / 256 : (p.N + BLOCK_N - 1) / BLOCK_N;
  long long grid = m_tiles_bound * n_tiles;
  // Tiles are drawn dynamically, so this kernel always asks for every SM: CTAs that find their
  // SM taken by a concurrent kernel start late and take fewer tiles.  (B200MOE_GEMM_HONOUR_LIMIT=1
  // makes it respect b200moe_set_cta_limit like the statically scheduled kernels.)
  static const bool honour = [] {
    const char* v = getenv("B200MOE_GEMM_HONOUR_LIMIT");
    return v != nullptr && v[0] == '1';
  }();
  const int sms = honour ? sm_count() : sm_count_device();
  if (grid > sms) grid = sms;
  if (grid < 1) grid = 1;
  GemmFp8Params q = p;
  q.sched_slot = sched_slot_of(stream);
  kern<<<(unsigned)grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, td, q);
  return launch_status();
}

}  // namespace b200

using namespace b200;

#ifdef B200_WAIT_TEST
// Test builds only (-DB200_WAIT_TEST=1, with a short -DB200_WAIT_LIMIT_CYCLES): when set, the
// producers of the next GEMM launches load nothing, so the bounded waits of the other roles run
// out, the kernel reports ERR_WAIT_TIMEOUT in the status block and returns.  Nothing traps,
// faults or spins without a limit; a launch after the flag is cleared runs normally.
static int g_withhold_loads = 0;
extern "C" int b200moe_debug_withhold_loads(int on) {
  g_withhold_loads = on ? 1 : 0;
  return B200MOE_OK;
}
#define B200_SET_WITHHOLD(params) (params).withhold_loads = g_withhold_loads
#else
#define B200_SET_WITHHOLD(params) do {} while (0)
#endif

#ifdef B200_GEMM_TRACE
static long long* g_trace_buffer = nullptr;
// Debug builds only: the device buffer (kTraceSlots * kTraceIts * kTraceFields int64) that CTA 0
// of the next GEMM launches writes its cycle stamps into; NULL switches the stamps off.
extern "C" int b200moe_debug_set_gemm_trace(long long* buffer) {
  g_trace_buffer = buffer;
  return B200MOE_OK;
}
extern "C" int b200moe_debug_gemm_trace_shape(int* slots, int* its, int* fields, int* first) {
  *slots = kTraceSlots; *its = kTraceIts; *fields = kTraceFields; *first = kTraceFirst;
  return B200MOE_OK;
}
#define B200_SET_TRACE(params) (params).trace = g_trace_buffer
#else
#define B200_SET_TRACE(params) do {} while (0)
#endif

// 1: the pair form whenever it can serve the call; -1 (default) and 0: the single-CTA form.
static std::atomic<int> g_pair_mode{[] {
  const char* v = getenv("B200MOE_GEMM_PAIR");
  return v == nullptr ? -1 : (v[0] == '0' ? 0 : 1);
}()};

extern "C" int b200moe_set_gemm_pair(int mode) {
  if (mode < -1 || mode > 1) return B200MOE_ERR_ARG;
  g_pair_mode.store(mode, std::memory_order_relaxed);
  return B200MOE_OK;
}

// The tensor map of the bf16 output for the epilogue's TMA stores (blocks of 32 rows x 32
// columns, 64-byte swizzle), or a copy of `fallback` when the output cannot leave that way:
// scattered rows, no plain output, B200MOE_GEMM_TMA_STORE=0.  Returns whether `td` describes d.
static bool output_tensor_map(CUtensorMap* td, const CUtensorMap& fallback, void* d, long long ldd, int N,
                              long long rows, bool eligible) {
  static const bool off = [] {
    const char* v = getenv("B200MOE_GEMM_TMA_STORE");
    return v != nullptr && v[0] == '0';
  }();
  *td = fallback;
  if (off || !eligible || d == nullptr || rows <= 0) return false;
  uint64_t dims[2] = {(uint64_t)N, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ldd * 2};
  uint32_t box[2] = {32, 32};
  CUtensorMap m;
  if (encode_tensor_map(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B) !=
      B200MOE_OK)
    return false;
  *td = m;
  return true;
}

// Shared by the plain product (d != NULL) and the one with the combine fused into its store
// (out_f32 != NULL).
static int grouped_gemm_fp8_impl(const void* a, long long lda, const float* a_scale, long long as_row_stride,
                                 long long as_kb_stride, const void* b, const float* b_scale, void* d,
                                 long long ldd, float* out_f32, long long ldo, long long tokens,
                                 const int32_t* row_token,
                                 const float* row_weight, const int32_t* row_map, const void* addend,
                                 long long ldc, const int32_t* offsets, int groups, int weights,
                                 long long rows_total, int N, int K, int b_mn_major, int block_n,
                                 int32_t* status, void* stream) {
  const bool fused = out_f32 != nullptr;
  if (!a || !a_scale || !b || !b_scale || !offsets || !status) return B200MOE_ERR_ARG;
  if (fused ? (!row_token || !row_weight || d != nullptr || tokens <= 0) : !d) return B200MOE_ERR_ARG;
  if (fused && (block_n != 256 || (ldo % 4) || ((uintptr_t)out_f32 & 15) || (N % 4))) return B200MOE_ERR_ALIGN;
  if (groups <= 0 || N <= 0 || K <= 0 || rows_total < 0) return B200MOE_ERR_ARG;
  if (weights <= 0 || groups % weights != 0) return B200MOE_ERR_ARG;
  if (groups > kMaxGroups || rows_total > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if (block_n != 128 && block_n != 256) return B200MOE_ERR_ARG;
  if ((N % 8) || (K % 16) || (lda % 16) || (ldd % 8)) return B200MOE_ERR_ALIGN;
  if (addend != nullptr && ((ldc % 8) || ((uintptr_t)addend & 15))) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)d & 15)) return B200MOE_ERR_ALIGN;
  if (b_mn_major && (N % 16)) return B200MOE_ERR_ALIGN;
  if (rows_total == 0) return B200MOE_OK;

  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)lda};
    uint32_t box[2] = {128, 128};
    int r = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  const int kblocks = (K + 127) / 128;
  const int nblocks = (N + 127) / 128;
  GemmFp8Params p;
  p.a_scale = a_scale;
  p.as_row_stride = as_row_stride;
  p.as_kb_stride = as_kb_stride;
  p.b_scale = b_scale;
  p.d = reinterpret_cast<__nv_bfloat16*>(d);
  p.ldd = ldd;
  static const bool narrow_store = [] {  // B200MOE_GEMM_WIDE_STORE=0: the store through shared memory
    const char* v = getenv("B200MOE_GEMM_WIDE_STORE");
    return v != nullptr && v[0] == '0';
  }();
  p.wide_store = (!narrow_store && d != nullptr && ((uintptr_t)d & 31) == 0 && (ldd % 16) == 0) ? 1 : 0;
  CUtensorMap td;
  p.tma_store = output_tensor_map(&td, ta, d, ldd, N, rows_total, !fused && row_map == nullptr) ? 1 : 0;
  p.addend = reinterpret_cast<const __nv_bfloat16*>(addend);
  p.ldc = ldc;
  p.offsets = offsets;
  p.groups = groups;
  p.N = N;
  p.K = K;
  p.rows_total = (int)rows_total;
  p.weights = weights;
  p.act_q = nullptr;
  p.ldq = 0;
  p.act_scale = nullptr;
  p.acts_row_stride = p.acts_kb_stride = 0;
  p.limit = 0.f;
  p.limited = 0;
  p.out_f32 = out_f32;
  p.ldo = ldo;
  p.row_token = row_token;
  p.row_weight = row_weight;
  p.row_map = row_map;
  p.out_rows = fused ? tokens : rows_total;
  p.status = status;
  B200_SET_TRACE(p);
  B200_SET_WITHHOLD(p);
  // The pair form (two CTAs per 256 x 256 tile) serves the plain and the scattered store of the
  // wide tile on request only (b200moe_set_gemm_pair(1) or B200MOE_GEMM_PAIR=1): it halves the
  // B traffic through shared memory, but its hand-backs cross the pair through mbarriers, and
  // measured 13-25% behind the single-CTA form, whose hand-backs are hardware barriers.
  const int pair_mode = g_pair_mode.load(std::memory_order_relaxed);
  static const bool pair_split = [] {  // B200MOE_GEMM_PAIR_SPLIT=1: each K block as two N=128 halves
    const char* v = getenv("B200MOE_GEMM_PAIR_SPLIT");
    return v != nullptr && v[0] == '1';
  }();
  const bool pair = !fused && block_n == 256 && pair_mode == 1 && sm_count() == sm_count_device();
  if (!b_mn_major) {
    // B is [groups, N, K], K contiguous; scales [groups, ceil(N/128), ceil(K/128)].
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)weights};
    uint64_t strides[2] = {(uint64_t)K, (uint64_t)K * (uint64_t)N};
    uint32_t box[3] = {128, pair ? (pair_split ? 64u : 128u) : (uint32_t)block_n, 1};
    int r = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
    p.bs_group_stride = (long long)nblocks * kblocks;
    p.bs_n_stride = kblocks;
    p.bs_k_stride = 1;
  } else {
    // B is [groups, K, N], N contiguous (the stored weight read for an input gradient);
    // scales [groups, ceil(K/128), ceil(N/128)].
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)weights};
    uint64_t strides[2] = {(uint64_t)N, (uint64_t)K * (uint64_t)N};
    // split pair form: 64 columns per CTA and half, as K-rows of 64 bytes (64-byte swizzle)
    uint32_t box[3] = {pair && pair_split ? 64u : 128u, 128, 1};
    int r = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, dims, strides, box,
                              pair && pair_split ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
    p.bs_group_stride = (long long)nblocks * kblocks;
    p.bs_n_stride = 1;
    p.bs_k_stride = nblocks;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (pair && pair_split)
    return b_mn_major ? launch_gemm_pair<true, true>(ta, tb, td, p, s) : launch_gemm_pair<false, true>(ta, tb, td, p, s);
  if (pair)
    return b_mn_major ? launch_gemm_pair<true, false>(ta, tb, td, p, s) : launch_gemm_pair<false, false>(ta, tb, td, p, s);
  // the 256-wide tile issues each K block in two halves (B200MOE_GEMM_SPLIT=0: in one piece)
  static const bool split = [] {
    const char* v = getenv("B200MOE_GEMM_SPLIT");
    return v == nullptr || v[0] != '0';
  }();
  if (fused) {
    if (split)
      return b_mn_major ? launch_gemm<256, true, 2, true>(ta, tb, td, p, s) : launch_gemm<256, false, 2, true>(ta, tb, td, p, s);
    return b_mn_major ? launch_gemm<256, true, 2>(ta, tb, td, p, s) : launch_gemm<256, false, 2>(ta, tb, td, p, s);
  }
  if (block_n == 128) {
    return b_mn_major ? launch_gemm<128, true>(ta, tb, td, p, s) : launch_gemm<128, false>(ta, tb, td, p, s);
  }
  if (split)
    return b_mn_major ? launch_gemm<256, true, 0, true>(ta, tb, td, p, s) : launch_gemm<256, false, 0, true>(ta, tb, td, p, s);
  return b_mn_major ? launch_gemm<256, true>(ta, tb, td, p, s) : launch_gemm<256, false>(ta, tb, td, p, s);
}

extern "C" int b200moe_grouped_gemm_fp8(const void* a, long long lda, const float* a_scale,
                                        long long as_row_stride, long long as_kb_stride, const void* b,
                                        const float* b_scale, void* d, long long ldd,
                                        const void* addend, long long ldc, const int32_t* offsets, int groups, int weights,
                                        long long rows_total, int N, int K, int b_mn_major, int block_n,
                                        int32_t* status, void* stream) {
  if (!d) return B200MOE_ERR_ARG;
  return grouped_gemm_fp8_impl(a, lda, a_scale, as_row_stride, as_kb_stride, b, b_scale, d, ldd, nullptr, 0, 0,
                               nullptr, nullptr, nullptr, addend, ldc, offsets, groups, weights, rows_total, N, K,
                               b_mn_major, block_n, status, stream);
}

// The same product with its rows stored where `row_map` says: d[row_map[r], :] = product[r, :].
// row_map must be a permutation of the rows that belong to a group (rows_total entries).
extern "C" int b200moe_grouped_gemm_fp8_scatter(const void* a, long long lda, const float* a_scale,
                                                long long as_row_stride, long long as_kb_stride, const void* b,
                                                const float* b_scale, void* d, long long ldd,
                                                const int32_t* row_map, const void* addend, long long ldc,
                                                const int32_t* offsets, int groups, int weights,
                                                long long rows_total, int N, int K, int b_mn_major, int block_n,
                                                int32_t* status, void* stream) {
  if (!d || !row_map) return B200MOE_ERR_ARG;
  return grouped_gemm_fp8_impl(a, lda, a_scale, as_row_stride, as_kb_stride, b, b_scale, d, ldd, nullptr, 0, 0,
                               nullptr, nullptr, row_map, addend, ldc, offsets, groups, weights, rows_total, N, K,
                               b_mn_major, block_n, status, stream);
}

// The down projection with the un-permute / combine fused into its store:
//   out_f32[row_token[r], :] += row_weight[r] * bf16(sum_k ... [r, :])   (16-byte fp32 atomics)
// out_f32 [tokens, N] must hold the starting value of every token row (zero, or the residual).
extern "C" int b200moe_grouped_gemm_fp8_combine(const void* a, long long lda, const float* a_scale,
                                                long long as_row_stride, long long as_kb_stride, const void* b,
                                                const float* b_scale, float* out_f32, long long ldo,
                                                long long tokens, const int32_t* row_token,
                                                const float* row_weight,
                                                const void* addend, long long ldc, const int32_t* offsets,
                                                int groups, int weights, long long rows_total, int N, int K,
                                                int b_mn_major, int32_t* status, void* stream) {
  if (!out_f32) return B200MOE_ERR_ARG;
  return grouped_gemm_fp8_impl(a, lda, a_scale, as_row_stride, as_kb_stride, b, b_scale, nullptr, 0, out_f32, ldo,
                               tokens, row_token, row_weight, nullptr, addend, ldc, offsets, groups, weights, rows_total,
                               N, K, b_mn_major, 256, status, stream);
}

// Up projection with the SwiGLU epilogue fused: h13 (bf16, gate columns then up columns, the
// residual the backward pass needs) and act = silu(gate) * up as E4M3 with 1x128 scales, in
// one kernel.  b is w13 [weights, 2F, K] (gate rows then up rows).
extern "C" int b200moe_grouped_gemm_fp8_swiglu(const void* a, long long lda, const float* a_scale,
                                               long long as_row_stride, long long as_kb_stride, const void* b,
                                               const float* b_scale, void* h13, long long ldh, void* act_q,
                                               long long ldq, float* act_scale, long long acts_row_stride,
                                               long long acts_block_stride, const int32_t* offsets, int groups,
                                               int weights, long long rows_total, int F, int K, float limit,
                                               int limited, int32_t* status, void* stream) {
  if (!a || !a_scale || !b || !b_scale || !h13 || !act_q || !act_scale || !offsets || !status)
    return B200MOE_ERR_ARG;
  if (groups <= 0 || F <= 0 || K <= 0 || rows_total < 0) return B200MOE_ERR_ARG;
  if (weights <= 0 || groups % weights != 0) return B200MOE_ERR_ARG;
  if (groups > kMaxGroups || rows_total > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((F % 128) || (K % 16) || (lda % 16) || (ldh % 8) || (ldq % 16)) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)h13 & 15) || ((uintptr_t)act_q & 15))
    return B200MOE_ERR_ALIGN;
  if (rows_total == 0) return B200MOE_OK;
  const int N = 2 * F;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)lda};
    uint32_t box[2] = {128, 128};
    int r = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)weights};
    uint64_t strides[2] = {(uint64_t)K, (uint64_t)K * (uint64_t)N};
    uint32_t box[3] = {128, 128, 1};  // 128 gate rows and 128 up rows are two loads per stage
    int r = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  const int kblocks = (K + 127) / 128;
  const int nblocks = N / 128;
  GemmFp8Params p;
  p.a_scale = a_scale;
  p.as_row_stride = as_row_stride;
  p.as_kb_stride = as_kb_stride;
  p.b_scale = b_scale;
  p.bs_group_stride = (long long)nblocks * kblocks;
  p.bs_n_stride = kblocks;
  p.bs_k_stride = 1;
  p.d = reinterpret_cast<__nv_bfloat16*>(h13);
  p.ldd = ldh;
  p.wide_store = (((uintptr_t)h13 & 31) == 0 && (ldh % 16) == 0) ? 1 : 0;
  CUtensorMap td;
  p.tma_store = output_tensor_map(&td, ta, h13, ldh, N, rows_total, true) ? 1 : 0;
  p.addend = nullptr;
  p.ldc = 0;
  p.offsets = offsets;
  p.groups = groups;
  p.N = N;
  p.K = K;
  p.rows_total = (int)rows_total;
  p.weights = weights;
  p.act_q = reinterpret_cast<uint8_t*>(act_q);
  p.ldq = ldq;
  p.act_scale = act_scale;
  p.acts_row_stride = acts_row_stride;
  p.acts_kb_stride = acts_block_stride;
  p.limit = limit;
  p.limited = limited;
  p.out_f32 = nullptr;
  p.ldo = 0;
  p.row_token = nullptr;
  p.row_weight = nullptr;
  p.row_map = nullptr;
  p.out_rows = rows_total;
  p.status = status;
  B200_SET_TRACE(p);
  B200_SET_WITHHOLD(p);
  return launch_gemm<256, false, 1>(ta, tb, td, p, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_set_cta_limit(int ctas) {
  if (ctas < 0) return B200MOE_ERR_ARG;
  set_cta_limit(ctas);
  return B200MOE_OK;
}
