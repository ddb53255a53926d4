// Grouped bf16 GEMM for sm_100a: the forward and input-gradient products of the bf16 compute
// path (weights kept or dequantised in bf16; reference: src/mlops/kernels/moe_grouped_gemm.py:
// 201-299, `grouped_mm_forward` / `grouped_mm_dgrad`):
//
//   D[rows of g, 0:N] = alpha * A[rows of g, 0:K] @ op(B[g])  (+ addend), bf16 out, fp32 sums
//
// A [rows, K] bf16 is K-major.  B is either [groups, N, K] (K-major: y = x W^T, the stored
// nn.Linear weight) or [groups, K, N] read MN-major (the SAME stored weight [out=K, in=N] for
// the input gradient dx = dy W: no transposed copy).  Groups are arbitrary row ranges of A
// (`offsets`); partial tiles are multiplied and masked at the store.
//
// Persistent kernel, one CTA per SM, 12 warps: TMA producer, one UMMA issuer, TMEM
// allocator, tile-table builder, eight epilogue warps.  Tile 128 x 256, K block 64 elements
// (128 bytes, 128-byte swizzle), 4 stages.  The sums of a tile stay in TMEM for the whole K
// loop (tcgen05.mma.kind::f16, M=128, N=256, K=16 per instruction); two 256-column accumulators,
// so a tile's drain and store overlap the next tile's multiplications.  Tiles are handed out
// by CTA index (static striding).
#include "common.cuh"
#include "host_util.h"

namespace b200 {

constexpr int kBfMaxGroups = 1024;
constexpr int kBfBlockM = 128;
constexpr int kBfBlockN = 256;
constexpr int kBfBlockK = 64;   // elements: 128 bytes
constexpr int kBfStages = 4;
constexpr int kBfThreads = 384;
constexpr int kBfABytes = kBfBlockM * kBfBlockK * 2;  // 16 KB
constexpr int kBfBBytes = kBfBlockN * kBfBlockK * 2;  // 32 KB
constexpr int kBfTileBytes = kBfStages * (kBfABytes + kBfBBytes);
constexpr int kBfBarBytes = 256;
constexpr int kBfSchedBytes = (2 * (kBfMaxGroups + 1) * 4 + 15) / 16 * 16;
constexpr int kBfStoreBytes = 8 * 32 * 80;
constexpr int kBfSmemBytes = 1024 + kBfTileBytes + kBfBarBytes + kBfSchedBytes + kBfStoreBytes + 1024;
constexpr int kBfTmemCols = 2 * kBfBlockN;

struct GemmBf16Params {
  __nv_bfloat16* d;
  long long ldd;
  const __nv_bfloat16* addend;  // optional [rows, N] term added in fp32 before the rounding
  long long ldc;
  const int* offsets;
  int groups, N, K, rows_total;
  int weights;  // group g multiplies weight matrix g % weights
  float alpha;  // d = alpha * (a @ op(b)) + addend
  int* status;
};

template <bool B_MN_MAJOR>
__global__ void __launch_bounds__(kBfThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmBf16Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kBfStages * kBfABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBfTileBytes);
  uint64_t* full = bars;                    // [stages] operands landed
  uint64_t* empty = bars + kBfStages;       // [stages] operands consumed
  uint64_t* tfull = bars + 2 * kBfStages;   // [2] accumulator complete
  uint64_t* tempty = bars + 2 * kBfStages + 2;  // [2] accumulator drained (eight epilogue warps)
  uint64_t* drain = bars + 2 * kBfStages + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kBfStages + 5);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* total_m_tiles_s = abort_flag + 1;
  int* m_tile_start = reinterpret_cast<int*>(smem + kBfTileBytes + kBfBarBytes);  // [groups+1]
  int* offs = m_tile_start + (kBfMaxGroups + 1);                                  // [groups+1]
  uint8_t* stage_base = smem + kBfTileBytes + kBfBarBytes + kBfSchedBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = p.groups;
  const int num_kb = (p.K + kBfBlockK - 1) / kBfBlockK;
  const int num_n_tiles = (p.N + kBfBlockN - 1) / kBfBlockN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBfStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kBfTmemCols);
    tmem_relinquish();
  }
  if (warp == 3) {
    // Tile table: exclusive scan of ceil(rows_g / 128) over the groups; a malformed row table
    // (negative, decreasing, past the end) is reported and leaves no tile.
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
      const int tiles = (g < groups && !bad) ? (hi - lo + kBfBlockM - 1) / kBfBlockM : 0;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
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
      if (bad) report_error(p.status, ERR_BAD_OFFSETS, 40, 0);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = (*total_m_tiles_s) * num_n_tiles;
  struct Tile {
    int group, m0, rows_valid, n0;
  };
  auto locate = [&](int t) {
    const int mt = t / num_n_tiles;
    int lo = 0, hi = groups - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (m_tile_start[mid] <= mt) lo = mid;
      else hi = mid - 1;
    }
    Tile c;
    c.group = lo;
    c.m0 = offs[lo] + (mt - m_tile_start[lo]) * kBfBlockM;
    c.rows_valid = min(kBfBlockM, offs[lo + 1] - c.m0);
    c.n0 = (t - mt * num_n_tiles) * kBfBlockN;
    return c;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile c = locate(t);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kBfStages;
          const uint32_t ph = (it / kBfStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 41)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[s], kBfABytes + kBfBBytes);
          tma_load_2d(sA + s * kBfABytes, &tmap_a, &full[s], kb * kBfBlockK, c.m0);
          if (!B_MN_MAJOR) {
            tma_load_3d(sB + s * kBfBBytes, &tmap_b, &full[s], kb * kBfBlockK, c.n0, c.group % p.weights);
          } else {
            // four panels of 64 columns (128 bytes) x 64 K-rows
#pragma unroll
            for (int panel = 0; panel < kBfBlockN / 64; ++panel)
              tma_load_3d(sB + s * kBfBBytes + panel * (64 * 128), &tmap_b, &full[s], c.n0 + panel * 64,
                          kb * kBfBlockK, c.group % p.weights);
          }
        }
      }
      if (!ok) {
        // Unwinding: give the copies that were issued a bounded chance to land before this
        // CTA's shared memory is released.
        for (int s = 0; s < kBfStages; ++s) {
          if (it <= (uint32_t)s) continue;
          const uint32_t last = ((it - 1 - s) / kBfStages) * kBfStages + s;
          const uint32_t ph = (last / kBfStages) & 1;
          const long long start = clock64();
          while (!mbar_try(&full[s], ph) && clock64() - start < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, 0, B_MN_MAJOR ? 1 : 0, kBfBlockM, kBfBlockN);
      uint32_t it = 0, tb = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tb) {
        const int buf = tb & 1;
        const uint32_t aph = (tb >> 1) & 1;
        if (!mbar_wait(&tempty[buf], aph ^ 1, abort_flag, p.status, 43)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kBfBlockN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kBfStages;
          const uint32_t ph = (it / kBfStages) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, 42)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + s * kBfABytes), 16, 1024);
          const uint32_t b_addr = smem_u32(sB + s * kBfBBytes);
          // K-major B: rows of 128 bytes, 32 bytes (16 elements) further per instruction.
          // MN-major B: panels of 64 columns, 8 KB apart; 16 K-rows of 128 bytes further.
          const uint64_t bdesc = B_MN_MAJOR ? make_smem_desc(b_addr, 64 * 128, 1024) : make_smem_desc(b_addr, 16, 1024);
          constexpr uint64_t kStepA = (uint64_t)(32 >> 4);
          constexpr uint64_t kStepB = (uint64_t)(B_MN_MAJOR ? ((16 * 128) >> 4) : (32 >> 4));
#pragma unroll
          for (int k = 0; k < kBfBlockK / 16; ++k)
            umma_f16(d_tmem, adesc + k * kStepA, bdesc + k * kStepB, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (kb == num_kb - 1) umma_commit(&tfull[buf]);
        }
      }
      if (!ok) {
        umma_commit(drain);
        const long long start = clock64();
        while (!mbar_try(drain, 0) && clock64() - start < 20000000LL) {}
      }
    }
  } else if (warp >= 4) {
    // ------------------------------- epilogue --------------------------------
    constexpr int kCols = kBfBlockN / 2;  // columns owned by one thread
    constexpr int kChunks = kCols / 32;
    constexpr int kStageRowBytes = 80;  // 64 bytes of data, padded against bank conflicts
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;   // which half of the tile's columns
    uint8_t* stage = stage_base + (warp - 4) * (32 * kStageRowBytes);
    uint32_t tb = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tb) {
      const Tile c = locate(t);
      const int buf = tb & 1;
      const uint32_t aph = (tb >> 1) & 1;
      if (!mbar_wait_warp(&tfull[buf], aph, abort_flag, p.status, 44)) { ok = false; break; }
      tc_fence_after_sync();
      const int grow = c.m0 + q * 32 + lane;
      const int rows_here = c.rows_valid - q * 32;  // rows of this warp that belong to the group
      const int col0 = c.n0 + half * kCols;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kBfBlockN + half * kCols;
#pragma unroll
      for (int cc = 0; cc < kChunks; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + cc * 32, r);
        tmem_ld_wait();
        if (cc == kChunks - 1) {
          // everything this warp needs of the accumulator is in registers: hand it back
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[buf]);
        }
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = p.alpha * __uint_as_float(r[j]);
        if (p.addend != nullptr && lane < rows_here) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + cc * 32 + j + 8 <= p.N) {
              const uint4 raw = *reinterpret_cast<const uint4*>(p.addend + (long long)grow * p.ldc + col0 + cc * 32 + j);
              const __nv_bfloat162* cv = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(cv[u]);
                acc[j + 2 * u] += f.x;
                acc[j + 2 * u + 1] += f.y;
              }
            }
          }
        }
        // The warp holds 32 rows x 32 columns, one row per lane.  Through a small per-warp
        // shared-memory buffer they leave as 8 rows x 64 contiguous bytes per instruction.
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          v.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
          v.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
          v.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
          v.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
          *reinterpret_cast<uint4*>(stage + lane * kStageRowBytes + j * 2) = v;
        }
        __syncwarp();
        const int piece = lane & 3;  // 16-byte piece of the 64-byte row slab
        const int col = col0 + cc * 32 + piece * 8;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + (lane >> 2);
          if (rr < rows_here && col + 8 <= p.N) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * kStageRowBytes + piece * 16);
            *reinterpret_cast<uint4*>(p.d + (long long)(c.m0 + q * 32 + rr) * p.ldd + col) = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kBfTmemCols);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200moe_grouped_gemm_bf16(const void* a, long long lda, const void* b, void* d, long long ldd,
                                         const void* addend, long long ldc, const int32_t* offsets, int groups,
                                         int weights, long long rows_total, int N, int K, int b_mn_major,
                                         float alpha, int32_t* status, void* stream) {
  if (!a || !b || !d || !offsets || !status) return B200MOE_ERR_ARG;
  if (groups <= 0 || weights <= 0 || groups % weights != 0 || N <= 0 || K <= 0 || rows_total < 0) return B200MOE_ERR_ARG;
  if (groups > kBfMaxGroups || rows_total > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldd % 8) || (addend && (ldc % 8))) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)d & 15) || ((uintptr_t)addend & 15))
    return B200MOE_ERR_ALIGN;
  if (rows_total == 0) return B200MOE_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {(uint32_t)kBfBlockK, (uint32_t)kBfBlockM};
    int r = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  if (!b_mn_major) {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)weights};
    uint64_t strides[2] = {(uint64_t)K * 2, (uint64_t)N * K * 2};
    uint32_t box[3] = {(uint32_t)kBfBlockK, (uint32_t)kBfBlockN, 1};
    int r = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  } else {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)weights};
    uint64_t strides[2] = {(uint64_t)N * 2, (uint64_t)N * K * 2};
    uint32_t box[3] = {64, (uint32_t)kBfBlockK, 1};
    int r = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  GemmBf16Params p;
  p.d = reinterpret_cast<__nv_bfloat16*>(d);
  p.ldd = ldd;
  p.addend = reinterpret_cast<const __nv_bfloat16*>(addend);
  p.ldc = ldc;
  p.offsets = offsets;
  p.groups = groups;
  p.N = N;
  p.K = K;
  p.rows_total = (int)rows_total;
  p.weights = weights;
  p.alpha = alpha;
  p.status = status;
  // upper bound of the tile count: every group may end in a partial tile
  const long long m_tiles = rows_total / kBfBlockM + groups;
  const long long tiles = m_tiles * ((N + kBfBlockN - 1) / kBfBlockN);
  long long grid = tiles < sm_count() ? tiles : sm_count();
  if (grid < 1) grid = 1;
  if (b_mn_major) {
    auto kern = grouped_gemm_bf16_kernel<true>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBfSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kBfThreads, kBfSmemBytes, s>>>(ta, tb, p);
  } else {
    auto kern = grouped_gemm_bf16_kernel<false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBfSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kBfThreads, kBfSmemBytes, s>>>(ta, tb, p);
  }
  return launch_status();
}
