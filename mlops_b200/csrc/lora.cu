// Rank-r side products of expert LoRA on expert-sorted rows (HBM-bound SIMT kernels; the
// rank is 8..64, so these products are a few percent of the layer's FLOPs):
//
//   lora_project : t[row, 0:r]  = x[row, 0:K] . W_e     (contraction over the wide axis K)
//   lora_expand  : c[row, 0:N]  = scale * t[row, 0:r] . W_e   (contraction over the rank)
//
// W_e is the factor of the row's expert, in either orientation, so the same two kernels
// serve the forward pass and the input gradients:
//   forward  up:   t1 = x A13^T (project, A13 [E,r,D] "rank-major"), c = s t1 B13^T (expand,
//                  B13 [E,2F,r] "wide-major"), c enters the base GEMM as an addend
//   backward:      dt = g B (project, B "wide-major"), dx = dt A (expand, A "rank-major")
// (reference: src/mlops/lora/experts.py:140-167, src/mlops/lora/grouped.py:19-110;
// the addend-before-SwiGLU form is that of src/mlops/providers/sonicmoe/lora.py:1062-1130).
// Factor gradients are grouped weight gradients with one narrow side and run on the
// tcgen05 weight-gradient kernel.
//
// A CTA owns a block of consecutive sorted rows (64 for ranks up to 16, fewer above); it
// walks the experts that own rows in that block, stages the expert's factor chunk in shared memory and lets each warp work on its rows.
#include "common.cuh"
#include "host_util.h"

namespace b200 {

constexpr int kLoraThreads = 256;
constexpr int kLoraChunk = 1024;  // wide-axis elements staged per step

__device__ __forceinline__ int expert_of_row(const int* offsets, int experts, int row) {
  int lo = 0, hi = experts - 1;  // last e with offsets[e] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offsets[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// rank_major != 0: W is [E, r, K] (K contiguous); else W is [E, K, r] (r contiguous).
template <int RMAX>
__global__ void __launch_bounds__(kLoraThreads)
lora_project_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                    int rank_major, const int* __restrict__ offsets, int experts, int rows, int K, int r,
                    __nv_bfloat16* __restrict__ t, long long ldt) {
  extern __shared__ __nv_bfloat16 sw[];  // [RMAX][kLoraChunk + 8]
  constexpr int kPitch = kLoraChunk + 8;
  constexpr int kRowsPerWarp = 128 / RMAX;  // keeps the per-thread sums at 128 registers
  constexpr int kLoraRows = kRowsPerWarp * (kLoraThreads / 32);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kLoraRows;
  const int row_end = min(row0 + kLoraRows, rows);
  const int e_first = expert_of_row(offsets, experts, row0);
  const int e_last = expert_of_row(offsets, experts, row_end - 1);
  for (int e = e_first; e <= e_last; ++e) {
    const int lo = max(offsets[e], row0), hi = min(offsets[e + 1], row_end);
    if (hi <= lo) continue;  // block-uniform
    float acc[kRowsPerWarp][RMAX];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i)
#pragma unroll
      for (int j = 0; j < RMAX; ++j) acc[i][j] = 0.f;
    const __nv_bfloat16* we = w + (long long)e * r * K;
    for (int k0 = 0; k0 < K; k0 += kLoraChunk) {
      const int kc = min(kLoraChunk, K - k0);
      __syncthreads();
      if (rank_major) {
        for (int idx = threadIdx.x * 8; idx < r * kLoraChunk; idx += kLoraThreads * 8) {
          const int j = idx / kLoraChunk, k = idx % kLoraChunk;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (k < kc) v = *reinterpret_cast<const uint4*>(we + (long long)j * K + k0 + k);
          *reinterpret_cast<uint4*>(sw + j * kPitch + k) = v;
        }
      } else {
        for (int idx = threadIdx.x; idx < r * kLoraChunk; idx += kLoraThreads) {
          const int k = idx / r, j = idx % r;
          sw[j * kPitch + k] = k < kc ? we[(long long)(k0 + k) * r + j] : __float2bfloat16(0.f);
        }
      }
      __syncthreads();
      // All rows of the warp load their 16 bytes first (independent loads in flight), then each
      // factor slice read from shared memory is used for every row.
      for (int k = lane * 8; k < kc; k += 256) {
        uint4 raw[kRowsPerWarp];
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
          const int row = row0 + warp * kRowsPerWarp + i;
          raw[i] = (row >= lo && row < hi) ? *reinterpret_cast<const uint4*>(x + (long long)row * ldx + k0 + k)
                                           : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < RMAX; ++j) {
          if (j < r) {
            const uint4 wraw = *reinterpret_cast<const uint4*>(sw + j * kPitch + k);
            const __nv_bfloat162* wv = reinterpret_cast<const __nv_bfloat162*>(&wraw);
            float wf[8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float2 f = __bfloat1622float2(wv[u]);
              wf[2 * u] = f.x;
              wf[2 * u + 1] = f.y;
            }
#pragma unroll
            for (int i = 0; i < kRowsPerWarp; ++i) {
              const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(xv[u]);
                acc[i][j] = fmaf(f.x, wf[2 * u], acc[i][j]);
                acc[i][j] = fmaf(f.y, wf[2 * u + 1], acc[i][j]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int row = row0 + warp * kRowsPerWarp + i;
      if (row < lo || row >= hi) continue;
#pragma unroll
      for (int j = 0; j < RMAX; ++j) {
        const float v = warp_sum(acc[i][j]);
        if (lane == (j & 31) && j < r) t[(long long)row * ldt + j] = __float2bfloat16(v);
      }
    }
  }
}

// wide_major != 0: W is [E, N, r] (r contiguous); else W is [E, r, N] (N contiguous).
template <int RMAX>
__global__ void __launch_bounds__(kLoraThreads)
lora_expand_kernel(const __nv_bfloat16* __restrict__ t, long long ldt, const __nv_bfloat16* __restrict__ w,
                   int wide_major, const int* __restrict__ offsets, int experts, int rows, int N, int r,
                   float scale, __nv_bfloat16* __restrict__ c, long long ldc) {
  extern __shared__ __nv_bfloat16 sw[];  // [RMAX][kLoraChunk + 8]
  constexpr int kPitch = kLoraChunk + 8;
  constexpr int kRowsPerWarp = 8;
  constexpr int kLoraRows = kRowsPerWarp * (kLoraThreads / 32);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kLoraRows;
  const int row_end = min(row0 + kLoraRows, rows);
  const int n0 = blockIdx.y * kLoraChunk;
  const int nc = min(kLoraChunk, N - n0);
  const int e_first = expert_of_row(offsets, experts, row0);
  const int e_last = expert_of_row(offsets, experts, row_end - 1);
  for (int e = e_first; e <= e_last; ++e) {
    const int lo = max(offsets[e], row0), hi = min(offsets[e + 1], row_end);
    if (hi <= lo) continue;
    const __nv_bfloat16* we = w + (long long)e * r * N;
    __syncthreads();
    if (!wide_major) {
      for (int idx = threadIdx.x * 8; idx < r * kLoraChunk; idx += kLoraThreads * 8) {
        const int j = idx / kLoraChunk, n = idx % kLoraChunk;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n < nc) v = *reinterpret_cast<const uint4*>(we + (long long)j * N + n0 + n);
        *reinterpret_cast<uint4*>(sw + j * kPitch + n) = v;
      }
    } else {
      for (int idx = threadIdx.x; idx < r * kLoraChunk; idx += kLoraThreads) {
        const int n = idx / r, j = idx % r;
        sw[j * kPitch + n] = n < nc ? we[(long long)(n0 + n) * r + j] : __float2bfloat16(0.f);
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int row = row0 + warp * kRowsPerWarp + i;
      if (row < lo || row >= hi) continue;
      float tv[RMAX];
#pragma unroll
      for (int j = 0; j < RMAX; ++j) tv[j] = j < r ? __bfloat162float(t[(long long)row * ldt + j]) * scale : 0.f;
      for (int n = lane * 8; n < nc; n += 256) {
        float out[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) out[u] = 0.f;
#pragma unroll
        for (int j = 0; j < RMAX; ++j) {
          if (j < r) {
            const uint4 wraw = *reinterpret_cast<const uint4*>(sw + j * kPitch + n);
            const __nv_bfloat162* wv = reinterpret_cast<const __nv_bfloat162*>(&wraw);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float2 f = __bfloat1622float2(wv[u]);
              out[2 * u] = fmaf(tv[j], f.x, out[2 * u]);
              out[2 * u + 1] = fmaf(tv[j], f.y, out[2 * u + 1]);
            }
          }
        }
        uint4 o;
        o.x = pack_bf16x2(out[0], out[1]);
        o.y = pack_bf16x2(out[2], out[3]);
        o.z = pack_bf16x2(out[4], out[5]);
        o.w = pack_bf16x2(out[6], out[7]);
        *reinterpret_cast<uint4*>(c + (long long)row * ldc + n0 + n) = o;
      }
    }
  }
}

constexpr int kLoraSmemBytes(int rmax) { return rmax * (kLoraChunk + 8) * 2; }

}  // namespace b200

using namespace b200;

extern "C" int b200moe_lora_project(const void* x, long long ldx, const void* w, int rank_major,
                                    const int32_t* offsets, int experts, long long rows, int K, int rank,
                                    void* t, long long ldt, void* stream) {
  if (!x || !w || !offsets || !t || experts <= 0 || rows < 0 || K <= 0 || rank <= 0) return B200MOE_ERR_ARG;
  if (rank > 64 || experts > 1024 || rows > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* tp = reinterpret_cast<__nv_bfloat16*>(t);
#define LAUNCH(RMAX)                                                                                   \
  do {                                                                                                 \
    auto kern = lora_project_kernel<RMAX>;                                                             \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLoraSmemBytes(RMAX))  \
        != cudaSuccess) return B200MOE_ERR_LAUNCH;                                                     \
    const int block_rows = (128 / RMAX) * (kLoraThreads / 32);                                         \
    const unsigned grid = (unsigned)((rows + block_rows - 1) / block_rows);                            \
    kern<<<grid, kLoraThreads, kLoraSmemBytes(RMAX), s>>>(xp, ldx, wp, rank_major, offsets, experts,   \
                                                         (int)rows, K, rank, tp, ldt);                 \
  } while (0)
  if (rank <= 16) LAUNCH(16);
  else if (rank <= 32) LAUNCH(32);
  else LAUNCH(64);
#undef LAUNCH
  return launch_status();
}

extern "C" int b200moe_lora_expand(const void* t, long long ldt, const void* w, int wide_major,
                                   const int32_t* offsets, int experts, long long rows, int N, int rank,
                                   float scale, void* c, long long ldc, void* stream) {
  if (!t || !w || !offsets || !c || experts <= 0 || rows < 0 || N <= 0 || rank <= 0) return B200MOE_ERR_ARG;
  if (rank > 64 || experts > 1024 || rows > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((N % 8) || (ldc % 8) || ((uintptr_t)c & 15) || ((uintptr_t)w & 15)) return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((N + kLoraChunk - 1) / kLoraChunk));
  const __nv_bfloat16* tp = reinterpret_cast<const __nv_bfloat16*>(t);
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(c);
#define LAUNCH(RMAX)                                                                                   \
  do {                                                                                                 \
    auto kern = lora_expand_kernel<RMAX>;                                                              \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLoraSmemBytes(RMAX))  \
        != cudaSuccess) return B200MOE_ERR_LAUNCH;                                                     \
    kern<<<grid, kLoraThreads, kLoraSmemBytes(RMAX), s>>>(tp, ldt, wp, wide_major, offsets, experts,   \
                                                         (int)rows, N, rank, scale, cp, ldc);          \
  } while (0)
  if (rank <= 16) LAUNCH(16);
  else if (rank <= 32) LAUNCH(32);
  else LAUNCH(64);
#undef LAUNCH
  return launch_status();
}
