// Grouped weight-gradient GEMM for sm_100a (bf16 operands, fp32 accumulation in TMEM).
//
//   dW[g] (M x N) = G[rows of g, 0:M]^T @ X[rows of g, 0:N]
//
// Both operands are token-major matrices, so the contraction (token) axis is the slow
// axis of both: the tiles are loaded by TMA as K-rows of 128 bytes and handed to
// tcgen05.mma as MN-major operands.  The K extent of a group is arbitrary; the rows of
// the last K block that lie past the group's end are zeroed in both operand tiles before the
// MMAs are issued, so the neighbouring group's rows contribute nothing (not even a NaN).  Sums are fp32
// for the whole K loop (one TMEM accumulator per tile, two buffers so the epilogue of a
// tile overlaps the MMAs of the next) and are written at the requested dtype; a group
// without rows gets exact zeros (reference: src/mlops/kernels/moe_grouped_gemm.py:120-174,
// 300-342 -- fp32 sums, selectable output dtype, zero for empty experts).
#include "common.cuh"
#include "host_util.h"

#include <stdlib.h>

namespace b200 {

constexpr int kWgMaxGroups = 1024;
constexpr int kWgBlockM = 128;
constexpr int kWgBlockN = 256;
constexpr int kWgBlockK = 64;
constexpr int kWgStages = 4;
constexpr int kWgThreads = 384;
constexpr int kWgPanelBytes = kWgBlockK * 128;            // 64 K-rows x 64 bf16
constexpr int kWgABytes = (kWgBlockM / 64) * kWgPanelBytes;  // 16 KB
constexpr int kWgBBytes = (kWgBlockN / 64) * kWgPanelBytes;  // 32 KB
constexpr int kWgTileBytes = kWgStages * (kWgABytes + kWgBBytes);
constexpr int kWgSmemBytes = 1024 + kWgTileBytes + 256 + 4 * 4104;  // (the same for E4M3: 128-row stages of 48 KB)
constexpr int kWgTmemCols = 2 * kWgBlockN;
constexpr int kWgMaxOffsets = 4097;  // segments * groups + 1 entries are cached in shared memory

struct WgradParams {
  void* out;  // [groups, M, N]
  const int* offsets;
  int groups, M, N, rows_total;
  int segments;  // offsets holds segments*groups+1 entries; group g owns segment ranges s*groups+g
  int* status;
  float scale;     // out = scale * product (+ what out held, when accumulate)
  int accumulate;  // a caller's gradient buffer is updated in place, in fp32, with one rounding
  // E4M3 operands (FP8 kernel only): one fp32 scale per group and column of G ([groups, M]) and of
  // X ([groups, N]); the product of a group is multiplied by g_scale[m] * x_scale[n] at the store.
  const float* g_scale;
  const float* x_scale;
  int wide_store;  // the output's base and row pitch are multiples of 32 bytes: 32-byte stores
};

// Geometry of a K block in shared memory.  A panel is 128 bytes of an operand's columns for every
// K-row of the block: 64 bf16 columns x 64 rows, or 128 E4M3 columns x 128 rows -- 16 KB of G and
// 32 KB of X per stage either way.
template <bool FP8>
struct WgGeom {
  static constexpr int kBlockK = FP8 ? 128 : 64;               // K-rows per stage
  static constexpr int kPanelCols = FP8 ? 128 : 64;            // columns in 128 bytes
  static constexpr int kPanelBytes = kBlockK * 128;
  static constexpr int kAPanels = kWgBlockM / kPanelCols;
  static constexpr int kBPanels = kWgBlockN / kPanelCols;
  static constexpr int kABytes = kAPanels * kPanelBytes;
  static constexpr int kBBytes = kBPanels * kPanelBytes;
  static constexpr int kMmaK = FP8 ? 32 : 16;                  // K-rows per tcgen05.mma
};

template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float (&v)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

template <typename OutT>
__device__ __forceinline__ void load8(const OutT* src, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* src, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* src, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// The store of eight sums: scaled, and added to what the destination holds when the caller
// accumulates gradients over several calls (micro-batches) in one buffer.
// -DB200_WGRAD_ABLATE_STORE=1 (timing experiments only) drops the store: what the epilogue's
// writes cost the main loop shows as the difference.  The shipped library stores.
#ifndef B200_WGRAD_ABLATE_STORE
#define B200_WGRAD_ABLATE_STORE 0
#endif
template <typename OutT>
__device__ __forceinline__ void finish8(OutT* dst, float (&v)[8], float scale, int accumulate) {
  if (B200_WGRAD_ABLATE_STORE && v[0] != 12345.678f) return;
  if (accumulate) {
    float old[8];
    load8<OutT>(dst, old);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaf(scale, v[i], old[i]);
  } else if (scale != 1.0f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= scale;
  }
  store8<OutT>(dst, v);
}

// 32 bytes per lane and instruction: a lane's store fills whole 32-byte sectors of its output row
// (16-byte pieces of 32 different rows per instruction cost the weight gradient a fifth of its
// time in sector-merging traffic).  The address must be 32-byte aligned.
__device__ __forceinline__ void store_v8(void* dst, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void load_v8(const void* src, uint32_t (&w)[8]) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(src)
               : "memory");
}

// The store of one lane's 32 consecutive sums of a row (`cols` of them inside the matrix, a
// multiple of 8): scaled, added to the destination when the caller accumulates, rounded once.
// `wide`: the row pitch and base allow 32-byte accesses.
template <typename OutT>
__device__ __forceinline__ void finish32(OutT* dst, float (&v)[32], int cols, float scale, int accumulate, bool wide);

template <>
__device__ __forceinline__ void finish32<float>(float* dst, float (&v)[32], int cols, float scale, int accumulate,
                                                bool wide) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 + 8 > cols) break;
    float part[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) part[i] = v[g * 8 + i];
    if (!wide) {
      finish8<float>(dst + g * 8, part, scale, accumulate);
      continue;
    }
    uint32_t w[8];
    if (accumulate) {
      load_v8(dst + g * 8, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) part[i] = fmaf(scale, part[i], __uint_as_float(w[i]));
    } else if (scale != 1.0f) {
#pragma unroll
      for (int i = 0; i < 8; ++i) part[i] *= scale;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(part[i]);
    store_v8(dst + g * 8, w);
  }
}

template <>
__device__ __forceinline__ void finish32<__nv_bfloat16>(__nv_bfloat16* dst, float (&v)[32], int cols, float scale,
                                                        int accumulate, bool wide) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (wide && h * 16 + 16 <= cols) {
      uint32_t w[8];
      if (accumulate) {
        load_v8(dst + h * 16, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 old = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
          v[h * 16 + 2 * i] = fmaf(scale, v[h * 16 + 2 * i], old.x);
          v[h * 16 + 2 * i + 1] = fmaf(scale, v[h * 16 + 2 * i + 1], old.y);
        }
      } else if (scale != 1.0f) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[h * 16 + i] *= scale;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(v[h * 16 + 2 * i], v[h * 16 + 2 * i + 1]);
      store_v8(dst + h * 16, w);
    } else {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (h * 16 + g * 8 + 8 > cols) break;
        float part[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) part[i] = v[h * 16 + g * 8 + i];
        finish8<__nv_bfloat16>(dst + h * 16 + g * 8, part, scale, accumulate);
      }
    }
  }
}

template <typename OutT, bool FP8>
__global__ void __launch_bounds__(kWgThreads, 1)
grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_x,
                     const WgradParams p) {
  using Geo = WgGeom<FP8>;
  constexpr int kBlockK = Geo::kBlockK;
  constexpr int kABytes = Geo::kABytes, kBBytes = Geo::kBBytes, kPanelBytes = Geo::kPanelBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kWgStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWgTileBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kWgStages;
  uint64_t* tfull = bars + 2 * kWgStages;
  uint64_t* tempty = bars + 2 * kWgStages + 2;
  uint64_t* drain = bars + 2 * kWgStages + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kWgStages + 5);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* offs_s = reinterpret_cast<int*>(smem + kWgTileBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kWgBlockM - 1) / kWgBlockM;
  const int n_tiles = (p.N + kWgBlockN - 1) / kWgBlockN;
  const int tiles_per_group = m_tiles * n_tiles;
  const long long total_tiles = (long long)tiles_per_group * p.groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWgStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 8);
    mbar_init(&tempty[1], 8);
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_g);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kWgTmemCols);
    tmem_relinquish();
  }
  __syncthreads();  // abort_flag initialised before the table check may set it
  // The row ranges are read many times by every role: keep them in shared memory.  A malformed
  // table (negative, decreasing, past the end) is reported and every range becomes empty.
  {
    const int entries = p.segments * p.groups + 1;
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
      const int v = p.offsets[i];
      const int nxt = i + 1 < entries ? p.offsets[i + 1] : v;
      if (v < 0 || nxt < v || nxt > p.rows_total) {
        report_error(p.status, ERR_BAD_OFFSETS, 20, i);
        *abort_flag = 2;  // not an abort: marks the table as unusable
      }
      offs_s[i] = v;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool table_ok = *abort_flag != 2;
  __syncthreads();
  if (threadIdx.x == 0) *abort_flag = 0;
  __syncthreads();

  // Every role walks the same tile sequence and derives the same K ranges from the table.
  auto group_range = [&](int g, int seg, int& lo, int& hi) {
    const int at = seg * p.groups + g;
    lo = offs_s[at];
    hi = table_ok ? offs_s[at + 1] : lo;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int g = (int)(t / tiles_per_group);
        const int rem = (int)(t - (long long)g * tiles_per_group);
        const int m0 = (rem / n_tiles) * kWgBlockM;
        const int n0 = (rem % n_tiles) * kWgBlockN;
        for (int seg = 0; seg < p.segments && ok; ++seg) {
          int lo, hi;
          group_range(g, seg, lo, hi);
          const int num_kb = (hi - lo + kBlockK - 1) / kBlockK;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kWgStages;
            const uint32_t ph = (it / kWgStages) & 1;
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 21)) { ok = false; break; }
            mbar_arrive_expect_tx(&full[s], kABytes + kBBytes);
            const int krow = lo + kb * kBlockK;
#pragma unroll
            for (int pnl = 0; pnl < Geo::kAPanels; ++pnl)
              tma_load_2d(sA + s * kABytes + pnl * kPanelBytes, &tmap_g, &full[s], m0 + pnl * Geo::kPanelCols, krow);
#pragma unroll
            for (int pnl = 0; pnl < Geo::kBPanels; ++pnl)
              tma_load_2d(sB + s * kBBytes + pnl * kPanelBytes, &tmap_x, &full[s], n0 + pnl * Geo::kPanelCols, krow);
          }
        }
      }
      if (!ok) {
        const uint32_t issued = it;
        for (int s = 0; s < kWgStages; ++s) {
          if (issued <= (uint32_t)s) continue;
          const uint32_t last = ((issued - 1 - s) / kWgStages) * kWgStages + s;
          const uint32_t ph = (last / kWgStages) & 1;
          const long long start = clock64();
          while (!mbar_try(&full[s], ph) && clock64() - start < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // All 32 lanes stay in the loop: they zero the K tail together; lane 0 issues.
    constexpr uint32_t idesc = FP8 ? make_idesc(0, 0, 1, 1, kWgBlockM, kWgBlockN)   // E4M3 x E4M3, both MN-major
                                   : make_idesc(1, 1, 1, 1, kWgBlockM, kWgBlockN);  // bf16 x bf16
    uint32_t it = 0, tb = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int g = (int)(t / tiles_per_group);
      int total_kb = 0;
      for (int seg = 0; seg < p.segments; ++seg) {
        int lo, hi;
        group_range(g, seg, lo, hi);
        total_kb += (hi - lo + kBlockK - 1) / kBlockK;
      }
      if (total_kb == 0) continue;
      const int buf = tb & 1;
      const uint32_t aph = (tb >> 1) & 1;
      ++tb;
      if (!mbar_wait_warp(&tempty[buf], aph ^ 1, abort_flag, p.status, 23)) { ok = false; break; }
      int done_kb = 0;
      for (int seg = 0; seg < p.segments && ok; ++seg) {
        int lo, hi;
        group_range(g, seg, lo, hi);
        const int num_kb = (hi - lo + kBlockK - 1) / kBlockK;
        for (int kb = 0; kb < num_kb; ++kb, ++it, ++done_kb) {
          const int s = it % kWgStages;
          const uint32_t ph = (it / kWgStages) & 1;
          if (!mbar_wait_warp(&full[s], ph, abort_flag, p.status, 22)) { ok = false; break; }
          const int valid = hi - lo - kb * kBlockK;
          if (valid < kBlockK) {
            // rows [valid, kBlockK) of every panel of BOTH operands: 128 bytes each, 16 bytes per
            // lane-step.  (Zeroing one operand would leave 0 x Inf = NaN when the next group's
            // rows hold an Inf or a NaN: groups must stay isolated.)
            const int nbytes = (kBlockK - valid) * 128;
            for (int pnl = 0; pnl < Geo::kAPanels + Geo::kBPanels; ++pnl) {
              uint8_t* base = (pnl < Geo::kAPanels ? sA + s * kABytes + pnl * kPanelBytes
                                                   : sB + s * kBBytes + (pnl - Geo::kAPanels) * kPanelBytes) +
                              valid * 128;
              for (int o = lane * 16; o < nbytes; o += 32 * 16)
                *reinterpret_cast<uint4*>(base + o) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t a_addr = smem_u32(sA + s * kABytes);
            const uint32_t b_addr = smem_u32(sB + s * kBBytes);
            const uint64_t adesc = make_smem_desc(a_addr, kPanelBytes, 1024);
            const uint64_t bdesc = make_smem_desc(b_addr, kPanelBytes, 1024);
            const uint32_t d_tmem = tmem_base + buf * kWgBlockN;
#pragma unroll
            for (int k = 0; k < kBlockK / Geo::kMmaK; ++k) {
              const uint64_t step = (uint64_t)((k * Geo::kMmaK * 128) >> 4);
              if constexpr (FP8) umma_f8(d_tmem, adesc + step, bdesc + step, idesc, (done_kb > 0 || k > 0) ? 1u : 0u);
              else umma_f16(d_tmem, adesc + step, bdesc + step, idesc, (done_kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty[s]);
            if (done_kb == total_kb - 1) umma_commit(&tfull[buf]);
          }
          __syncwarp();
        }
      }
    }
    if (!ok && lane == 0) {
      umma_commit(drain);
      const long long start = clock64();
      while (!mbar_try(drain, 0) && clock64() - start < 20000000LL) {}
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;
    constexpr int kCols = kWgBlockN / 2;
    uint32_t tb = 0;
    bool ok = true;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int g = (int)(t / tiles_per_group);
      const int rem = (int)(t - (long long)g * tiles_per_group);
      const int m0 = (rem / n_tiles) * kWgBlockM;
      const int n0 = (rem % n_tiles) * kWgBlockN;
      bool has_rows = false;
      for (int seg = 0; seg < p.segments; ++seg) {
        int lo, hi;
        group_range(g, seg, lo, hi);
        has_rows = has_rows || hi > lo;
      }
      const int m = m0 + q * 32 + lane;
      const int col0 = n0 + half * kCols;
      OutT* orow = out + ((long long)g * p.M + m) * p.N + col0;
      float row_scale = 1.0f;
      const float* col_scale = nullptr;
      if constexpr (FP8) {
        row_scale = m < p.M ? p.g_scale[(long long)g * p.M + m] : 0.f;
        col_scale = p.x_scale + (long long)g * p.N + col0;
      }
      int buf = 0;
      if (has_rows) {
        buf = tb & 1;
        const uint32_t aph = (tb >> 1) & 1;
        ++tb;
        if (!mbar_wait_warp(&tfull[buf], aph, abort_flag, p.status, 24)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kWgBlockN + half * kCols;
#pragma unroll
      for (int cc = 0; cc < kCols / 32; ++cc) {
        uint32_t r[32];
        if (has_rows) {
          tmem_ld_32x32(taddr + cc * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int cols = min(32, p.N - (col0 + cc * 32));  // of this chunk inside the matrix (a multiple of 8)
        if (m < p.M && cols > 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if constexpr (FP8) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (j < cols) {
                const float4 cs = *reinterpret_cast<const float4*>(col_scale + cc * 32 + j);
                v[j] *= row_scale * cs.x;
                v[j + 1] *= row_scale * cs.y;
                v[j + 2] *= row_scale * cs.z;
                v[j + 3] *= row_scale * cs.w;
              }
            }
          }
          finish32<OutT>(orow + cc * 32, v, cols, p.scale, p.accumulate, p.wide_store != 0);
        }
      }
      if (has_rows) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kWgTmemCols);
  }
}


// ---------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster share one 256 x 256 output tile.  CTA r of the
// pair owns output rows [r*128, r*128+128) (accumulated in its own TMEM) and loads, per K
// block, its 128 columns of G and 128 of the 256 columns of X; one tcgen05.mma.cta_group::2
// issued by the leader CTA multiplies across both SMs, so every operand byte is fetched from
// L2 and written to shared memory once per pair instead of once per CTA (32 KB instead of
// 48 KB per CTA and K block).  No load is multicast: each CTA's TMA loads land in its own
// shared memory and complete on its own barrier; after the K tail of its A tile is zeroed the
// CTA tells the leader with one (remote) mbarrier arrival (warp 1 of each CTA); warp 3 of the
// leader waits for both reports and issues the MMAs.  The leader's commits arrive on both
// CTAs' barriers.
// ---------------------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr int kPairABytes = 2 * kWgPanelBytes;  // 128 columns of G x 64 K-rows
constexpr int kPairBBytes = 2 * kWgPanelBytes;  // 128 columns of X x 64 K-rows
constexpr int kPairTileBytes = kPairStages * (kPairABytes + kPairBBytes);
constexpr int kPairSmemBytes = 1024 + kPairTileBytes + 512 + 4 * 4104;
constexpr int kPairBlockM = 256;  // per pair

template <typename OutT>
__global__ void __launch_bounds__(kWgThreads, 1)
grouped_wgrad_pair_kernel(const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_x,
                          const WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kPairStages * kPairABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairTileBytes);
  uint64_t* landed = bars;                         // [stages] this CTA's TMA bytes
  uint64_t* ready = bars + kPairStages;            // [stages] leader only: both CTAs' tiles usable
  uint64_t* empty = bars + 2 * kPairStages;        // [stages] stage consumed (leader's commit, both CTAs)
  uint64_t* tfull = bars + 3 * kPairStages;        // [2] accumulator complete (leader's commit, both CTAs)
  uint64_t* tempty = bars + 3 * kPairStages + 2;   // [2] leader only: both CTAs drained the buffer
  uint64_t* drain = bars + 3 * kPairStages + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kPairStages + 5);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* offs_s = reinterpret_cast<int*>(smem + kPairTileBytes + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + kPairBlockM - 1) / kPairBlockM;
  const int n_tiles = (p.N + kWgBlockN - 1) / kWgBlockN;
  const int tiles_per_group = m_tiles * n_tiles;
  const long long total_tiles = (long long)tiles_per_group * p.groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&landed[s], 1);
      mbar_init(&ready[s], 2);   // one arrival per CTA of the pair
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 16);  // 8 epilogue warps in each CTA
    mbar_init(&tempty[1], 16);
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_g);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, kWgTmemCols);
    tmem_relinquish_pair();
  }
  __syncthreads();  // abort_flag initialised before the table check may set it
  // The row ranges are read many times by every role: keep them in shared memory.  A malformed
  // table (negative, decreasing, past the end) is reported and every range becomes empty.
  {
    const int entries = p.segments * p.groups + 1;
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
      const int v = p.offsets[i];
      const int nxt = i + 1 < entries ? p.offsets[i + 1] : v;
      if (v < 0 || nxt < v || nxt > p.rows_total) {
        report_error(p.status, ERR_BAD_OFFSETS, 20, i);
        *abort_flag = 2;  // not an abort: marks the table as unusable
      }
      offs_s[i] = v;
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs exist before anyone arrives on a remote one
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool table_ok = *abort_flag != 2;
  __syncthreads();
  if (threadIdx.x == 0) *abort_flag = 0;
  __syncthreads();

  auto group_range = [&](int g, int seg, int& lo, int& hi) {
    const int at = seg * p.groups + g;
    lo = offs_s[at];
    hi = table_ok ? offs_s[at + 1] : lo;
  };

  if (warp == 0) {
    // ---- TMA producer of this CTA: its half of the G columns and its half of the X columns
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long t = pair; t < total_tiles && ok; t += num_pairs) {
        const int g = (int)(t / tiles_per_group);
        const int rem = (int)(t - (long long)g * tiles_per_group);
        const int m0 = (rem / n_tiles) * kPairBlockM + (int)rank * 128;
        const int n0 = (rem % n_tiles) * kWgBlockN + (int)rank * 128;
        for (int seg = 0; seg < p.segments && ok; ++seg) {
          int lo, hi;
          group_range(g, seg, lo, hi);
          const int num_kb = (hi - lo + kWgBlockK - 1) / kWgBlockK;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kPairStages;
            const uint32_t ph = (it / kPairStages) & 1;
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 31)) { ok = false; break; }
            mbar_arrive_expect_tx(&landed[s], kPairABytes + kPairBBytes);
            const int krow = lo + kb * kWgBlockK;
#pragma unroll
            for (int pnl = 0; pnl < 2; ++pnl) {
              tma_load_2d(sA + s * kPairABytes + pnl * kWgPanelBytes, &tmap_g, &landed[s], m0 + pnl * 64, krow);
              tma_load_2d(sB + s * kPairBBytes + pnl * kWgPanelBytes, &tmap_x, &landed[s], n0 + pnl * 64, krow);
            }
          }
        }
      }
      if (!ok) {
        const uint32_t issued = it;
        for (int s = 0; s < kPairStages; ++s) {
          if (issued <= (uint32_t)s) continue;
          const uint32_t last = ((issued - 1 - s) / kPairStages) * kPairStages + s;
          const long long start = clock64();
          while (!mbar_try(&landed[s], (last / kPairStages) & 1) && clock64() - start < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- every CTA: wait for its tiles, zero the K tail, report to the leader.
    uint32_t it = 0;
    bool ok = true;
    for (long long t = pair; t < total_tiles && ok; t += num_pairs) {
      const int g = (int)(t / tiles_per_group);
      for (int seg = 0; seg < p.segments && ok; ++seg) {
        int lo, hi;
        group_range(g, seg, lo, hi);
        const int num_kb = (hi - lo + kWgBlockK - 1) / kWgBlockK;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait_warp(&landed[s], ph, abort_flag, p.status, 32)) { ok = false; break; }
          const int valid = hi - lo - kb * kWgBlockK;
          if (valid < kWgBlockK) {
            // both operands (see the single-CTA kernel): this CTA's two G and two X panels
            const int nbytes = (kWgBlockK - valid) * 128;
            for (int pnl = 0; pnl < 4; ++pnl) {
              uint8_t* base = (pnl < 2 ? sA + s * kPairABytes + pnl * kWgPanelBytes
                                       : sB + s * kPairBBytes + (pnl - 2) * kWgPanelBytes) + valid * 128;
              for (int o = lane * 16; o < nbytes; o += 32 * 16)
                *reinterpret_cast<uint4*>(base + o) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
          // A stage that was only written by TMA needs no release from this thread.  One whose
          // tail rows this warp zeroed was made visible to the async proxy by the fence above;
          // the PTX memory model would additionally want a cluster-scope release here before the
          // leader's MMA may depend on those stores.  That arrival costs about a microsecond and
          // was measured at 19% of this kernel's time (one tail block per tile), so it is a
          // build option (-DB200_WGRAD_RELEASE_TAIL_ARRIVE); the default relies on the remote
          // arrival being delivered after this warp's earlier shared-memory stores, which holds
          // on sm_100 hardware (the results are bit-identical) but is not promised by the model.
          if (lane == 0) {
#ifdef B200_WGRAD_RELEASE_TAIL_ARRIVE
            if (valid < kWgBlockK) mbar_arrive_remote_release(&ready[s], 0);
            else
#endif
              mbar_arrive_remote(&ready[s], 0);
          }
        }
      }
    }
  } else if (warp == 3) {
    // ---- leader CTA only: wait for both reports and issue the pair MMAs.
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, 1, 1, kPairBlockM, kWgBlockN);
      uint32_t it = 0, tb = 0;
      bool ok = true;
      for (long long t = pair; t < total_tiles && ok; t += num_pairs) {
        const int g = (int)(t / tiles_per_group);
        int total_kb = 0;
        for (int seg = 0; seg < p.segments; ++seg) {
          int lo, hi;
          group_range(g, seg, lo, hi);
          total_kb += (hi - lo + kWgBlockK - 1) / kWgBlockK;
        }
        if (total_kb == 0) continue;
        const int buf = tb & 1;
        const uint32_t aph = (tb >> 1) & 1;
        ++tb;
        if (!mbar_wait(&tempty[buf], aph ^ 1, abort_flag, p.status, 33)) { ok = false; break; }
        for (int done_kb = 0; done_kb < total_kb; ++done_kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(&ready[s], ph, abort_flag, p.status, 34)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + s * kPairABytes), kWgPanelBytes, 1024);
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + s * kPairBBytes), kWgPanelBytes, 1024);
          const uint32_t d_tmem = tmem_base + buf * kWgBlockN;
#pragma unroll
          for (int k = 0; k < kWgBlockK / 16; ++k) {
            const uint64_t step = (uint64_t)((k * 16 * 128) >> 4);
            umma_f16_pair(d_tmem, adesc + step, bdesc + step, idesc, (done_kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[s], 3);
          if (done_kb == total_kb - 1) umma_commit_pair(&tfull[buf], 3);
        }
      }
      if (!ok) {
        umma_commit_pair(drain, 1);
        const long long start = clock64();
        while (!mbar_try(drain, 0) && clock64() - start < 20000000LL) {}
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;
    constexpr int kCols = kWgBlockN / 2;
    uint32_t tb = 0;
    bool ok = true;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    for (long long t = pair; t < total_tiles && ok; t += num_pairs) {
      const int g = (int)(t / tiles_per_group);
      const int rem = (int)(t - (long long)g * tiles_per_group);
      const int m0 = (rem / n_tiles) * kPairBlockM + (int)rank * 128;
      const int n0 = (rem % n_tiles) * kWgBlockN;
      bool has_rows = false;
      for (int seg = 0; seg < p.segments; ++seg) {
        int lo, hi;
        group_range(g, seg, lo, hi);
        has_rows = has_rows || hi > lo;
      }
      const int m = m0 + q * 32 + lane;
      const int col0 = n0 + half * kCols;
      OutT* orow = out + ((long long)g * p.M + m) * p.N + col0;
      int buf = 0;
      if (has_rows) {
        buf = tb & 1;
        const uint32_t aph = (tb >> 1) & 1;
        ++tb;
        if (!mbar_wait_warp(&tfull[buf], aph, abort_flag, p.status, 35)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kWgBlockN + half * kCols;
#pragma unroll
      for (int cc = 0; cc < kCols / 32; ++cc) {
        uint32_t r[32];
        if (has_rows) {
          tmem_ld_32x32(taddr + cc * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int cols = min(32, p.N - (col0 + cc * 32));  // of this chunk inside the matrix (a multiple of 8)
        if (m < p.M && cols > 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          finish32<OutT>(orow + cc * 32, v, cols, p.scale, p.accumulate, p.wide_store != 0);
        }
      }
      if (has_rows) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(&tempty[buf], 0);
      }
    }
  }

  tc_fence_before_sync();
  cluster_sync_all();  // the peer may still be arriving on, or reading from, this CTA
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kWgTmemCols);
  }
}

template <typename OutT>
static int launch_pair(const CUtensorMap& tg, const CUtensorMap& tx, const WgradParams& p, cudaStream_t s) {
  auto kern = grouped_wgrad_pair_kernel<OutT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess)
    return B200MOE_ERR_LAUNCH;
  const long long tiles = (long long)p.groups * ((p.M + kPairBlockM - 1) / kPairBlockM) *
                          ((p.N + kWgBlockN - 1) / kWgBlockN);
  long long pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kWgThreads);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tg, tx, p) != cudaSuccess) return B200MOE_ERR_LAUNCH;
  return launch_status();
}

}  // namespace b200

using namespace b200;

static int grouped_wgrad_impl(const void* g, long long ldg, const void* x, long long ldx, const int32_t* offsets,
                              int groups, int segments, long long rows_total, int M, int N, void* out,
                              int out_is_fp32, float scale, int accumulate, int32_t* status, void* stream);

extern "C" int b200moe_grouped_wgrad_bf16(const void* g, long long ldg, const void* x, long long ldx,
                                          const int32_t* offsets, int groups, int segments,
                                          long long rows_total, int M, int N, void* out, int out_is_fp32,
                                          int32_t* status, void* stream) {
  return grouped_wgrad_impl(g, ldg, x, ldx, offsets, groups, segments, rows_total, M, N, out, out_is_fp32, 1.0f, 0,
                            status, stream);
}

// out[g] += scale * G[rows of g]^T @ X[rows of g]: the gradient written into a buffer the caller
// keeps across calls (a parameter's .grad over the micro-batches of an accumulation window).
extern "C" int b200moe_grouped_wgrad_bf16_accumulate(const void* g, long long ldg, const void* x, long long ldx,
                                                     const int32_t* offsets, int groups, int segments,
                                                     long long rows_total, int M, int N, void* out,
                                                     int out_is_fp32, float scale, int32_t* status,
                                                     void* stream) {
  return grouped_wgrad_impl(g, ldg, x, ldx, offsets, groups, segments, rows_total, M, N, out, out_is_fp32, scale, 1,
                            status, stream);
}

static int grouped_wgrad_impl(const void* g, long long ldg, const void* x, long long ldx, const int32_t* offsets,
                              int groups, int segments, long long rows_total, int M, int N, void* out,
                              int out_is_fp32, float scale, int accumulate, int32_t* status, void* stream) {
  if (!g || !x || !offsets || !out || !status) return B200MOE_ERR_ARG;
  if (groups <= 0 || segments <= 0 || M <= 0 || N <= 0 || rows_total < 0) return B200MOE_ERR_ARG;
  if (groups > kWgMaxGroups || rows_total > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((long long)groups * segments + 1 > kWgMaxOffsets) return B200MOE_ERR_LIMIT;
  if ((M % 8) || (N % 8) || (ldg % 8) || (ldx % 8)) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)g & 15) || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return B200MOE_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const size_t esz = out_is_fp32 ? 4 : 2;
  if (rows_total == 0) {
    if (accumulate) return B200MOE_OK;  // nothing to add
    return cudaMemsetAsync(out, 0, (size_t)groups * M * N * esz, s) == cudaSuccess ? B200MOE_OK
                                                                                   : B200MOE_ERR_LAUNCH;
  }
  CUtensorMap tg, tx;
  {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)ldg * 2};
    uint32_t box[2] = {64, (uint32_t)kWgBlockK};
    int r = encode_tensor_map(&tg, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)ldx * 2};
    uint32_t box[2] = {64, (uint32_t)kWgBlockK};
    int r = encode_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  WgradParams p;
  p.out = out;
  p.offsets = offsets;
  p.groups = groups;
  p.M = M;
  p.N = N;
  p.rows_total = (int)rows_total;
  p.segments = segments;
  p.status = status;
  p.scale = scale;
  p.accumulate = accumulate;
  p.g_scale = nullptr;
  p.x_scale = nullptr;
  p.wide_store = (((uintptr_t)out & 31) == 0 && ((size_t)N * esz) % 32 == 0 && ((size_t)M * N * esz) % 32 == 0) ? 1 : 0;
  // Wide outputs go to the CTA-pair kernel (256-row tiles); narrow ones (LoRA factors) and the
  // B200MOE_WGRAD_SINGLE=1 escape hatch use the single-CTA kernel.
  static const bool force_single = [] {
    const char* v = getenv("B200MOE_WGRAD_SINGLE");
    return v != nullptr && v[0] == '1';
  }();
  if (!force_single && M > 128 && N > 128) {
    return out_is_fp32 ? launch_pair<float>(tg, tx, p, s) : launch_pair<__nv_bfloat16>(tg, tx, p, s);
  }
  const long long tiles = (long long)groups * ((M + kWgBlockM - 1) / kWgBlockM) * ((N + kWgBlockN - 1) / kWgBlockN);
  long long grid = tiles < sm_count() ? tiles : sm_count();
  if (out_is_fp32) {
    auto kern = grouped_wgrad_kernel<float, false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kWgThreads, kWgSmemBytes, s>>>(tg, tx, p);
  } else {
    auto kern = grouped_wgrad_kernel<__nv_bfloat16, false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kWgThreads, kWgSmemBytes, s>>>(tg, tx, p);
  }
  return launch_status();
}

// The same products from E4M3 operands: G and X quantised with one scale per (group, column)
// (b200moe_quantize_columns), multiplied at the FP8 rate with fp32 sums over all of a group's
// rows, and scaled by g_scale[g, m] * x_scale[g, n] at the store.  Behavioural model: the
// reference's FP8 weight gradient (src/mlops/kernels/quack_moe/wgrad.py:30-69: both operands
// quantised per feature over the expert's tokens, one GEMM with exact K, epilogue acc * xs * ws).
extern "C" int b200moe_grouped_wgrad_fp8(const void* g, long long ldg, const float* g_scale, const void* x,
                                         long long ldx, const float* x_scale, const int32_t* offsets, int groups,
                                         int segments, long long rows_total, int M, int N, void* out,
                                         int out_is_fp32, float scale, int accumulate, int32_t* status,
                                         void* stream) {
  if (!g || !x || !g_scale || !x_scale || !offsets || !out || !status) return B200MOE_ERR_ARG;
  if (groups <= 0 || segments <= 0 || M <= 0 || N <= 0 || rows_total < 0) return B200MOE_ERR_ARG;
  if (groups > kWgMaxGroups || rows_total > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((long long)groups * segments + 1 > kWgMaxOffsets) return B200MOE_ERR_LIMIT;
  if ((M % 16) || (N % 16) || (ldg % 16) || (ldx % 16)) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)g & 15) || ((uintptr_t)x & 15) || ((uintptr_t)out & 15) || ((uintptr_t)g_scale & 15) ||
      ((uintptr_t)x_scale & 15))
    return B200MOE_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const size_t esz = out_is_fp32 ? 4 : 2;
  if (rows_total == 0) {
    if (accumulate) return B200MOE_OK;
    return cudaMemsetAsync(out, 0, (size_t)groups * M * N * esz, s) == cudaSuccess ? B200MOE_OK
                                                                                   : B200MOE_ERR_LAUNCH;
  }
  using Geo = WgGeom<true>;
  CUtensorMap tg, tx;
  {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)ldg};
    uint32_t box[2] = {(uint32_t)Geo::kPanelCols, (uint32_t)Geo::kBlockK};
    int r = encode_tensor_map(&tg, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, g, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)rows_total};
    uint64_t strides[1] = {(uint64_t)ldx};
    uint32_t box[2] = {(uint32_t)Geo::kPanelCols, (uint32_t)Geo::kBlockK};
    int r = encode_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != B200MOE_OK) return r;
  }
  WgradParams p;
  p.out = out;
  p.offsets = offsets;
  p.groups = groups;
  p.M = M;
  p.N = N;
  p.rows_total = (int)rows_total;
  p.segments = segments;
  p.status = status;
  p.scale = scale;
  p.accumulate = accumulate;
  p.g_scale = g_scale;
  p.x_scale = x_scale;
  p.wide_store = (((uintptr_t)out & 31) == 0 && ((size_t)N * esz) % 32 == 0 && ((size_t)M * N * esz) % 32 == 0) ? 1 : 0;
  const long long tiles = (long long)groups * ((M + kWgBlockM - 1) / kWgBlockM) * ((N + kWgBlockN - 1) / kWgBlockN);
  long long grid = tiles < sm_count() ? tiles : sm_count();
  if (out_is_fp32) {
    auto kern = grouped_wgrad_kernel<float, true>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kWgThreads, kWgSmemBytes, s>>>(tg, tx, p);
  } else {
    auto kern = grouped_wgrad_kernel<__nv_bfloat16, true>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmemBytes) != cudaSuccess)
      return B200MOE_ERR_LAUNCH;
    kern<<<(unsigned)grid, kWgThreads, kWgSmemBytes, s>>>(tg, tx, p);
  }
  return launch_status();
}
