// Router top-k selection and the expert-sorted permutation, as integer-exact CUDA.
//
// route_topk: one warp per token.  Lane l holds experts l, l+32, l+64, ...; the K
// winners are found by K warp-wide arg-max rounds over (selection value, expert id)
// with ties going to the lowest expert id, which is the order a stable descending
// sort produces (reference: src/mlops/kernels/moe_router.py:290-344, the Triton
// twin :106-171).  Modes:
//   0 topk_then_softmax   select on logits, weights = softmax over the K picked logits
//   1 softmax_then_topk   select on logits (softmax is monotone), weights = softmax[id]
//   2 sigmoid_noaux_tc    select on sigmoid(logit)+bias inside the top `topk_group`
//                         groups (group score = sum of the group's two best selection
//                         values), weights = score[id] / sum(picked scores) * scaling
//
// sort_assignments: stable counting sort of the flat [T*K] expert ids
// (reference: src/mlops/kernels/moe_dispatch.py:106-119):
//   order[j]   flat assignment index (token*K + slot) held by sorted row j
//   offsets[e] first sorted row of expert e (offsets[E] = T*K)
//   slots[i]   sorted row of flat assignment i (the inverse permutation)
// Three launches: per-chunk histogram, scan (over chunks, then experts), ranked scatter.
#include "common.cuh"
#include "host_util.h"

namespace b200 {

constexpr int kRouteWarps = 8;
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortChunk = 4096;

struct Cand {
  float v;   // selection value
  int e;     // expert id
  float s;   // payload: the value the route weight is computed from
};

// The order of a stable descending torch.sort: NaN ranks above every number (and NaNs
// among themselves by index), equal values go to the lower expert id.  A row of NaN logits
// therefore still yields K distinct in-range ids, as the reference's sort does; the NaN
// shows up in the route weights and the output, never in an index.
__device__ __forceinline__ bool value_above(float v, float v2) {
  const bool n1 = v != v, n2 = v2 != v2;
  return (n1 || n2) ? (n1 && !n2) : (v > v2);
}
__device__ __forceinline__ bool better(float v, int e, float v2, int e2) {
  const bool n1 = v != v, n2 = v2 != v2;
  if (n1 || n2) return n1 && (!n2 || e < e2);
  return (v > v2) || (v == v2 && e < e2);
}
__device__ __forceinline__ float max_nan_high(float a, float b) { return value_above(b, a) ? b : a; }
__device__ __forceinline__ float min_nan_high(float a, float b) { return value_above(b, a) ? a : b; }

__device__ __forceinline__ Cand warp_argmax(Cand c) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, c.v, o);
    const int e2 = __shfl_xor_sync(0xffffffffu, c.e, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, c.s, o);
    if (better(v2, e2, c.v, c.e)) {
      c.v = v2;
      c.e = e2;
      c.s = s2;
    }
  }
  return c;
}

template <int EPL>
__global__ void __launch_bounds__(kRouteWarps * 32)
route_topk_kernel(const float* __restrict__ logits, long long ld, int T, int E, int K, int mode,
                  const float* __restrict__ bias, int n_group, int topk_group, float routed_scaling,
                  float* __restrict__ weights, int* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + (threadIdx.x >> 5);
  if (t >= T) return;
  const float NEG_INF = __int_as_float(0xff800000);

  float x[EPL], sel[EPL], pay[EPL];
  const float* row = logits + (long long)t * ld;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int e = j * 32 + lane;
    x[j] = e < E ? row[e] : NEG_INF;
  }

  if (mode == 2) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      const float sc = __fdiv_rn(1.0f, 1.0f + expf(-x[j]));
      pay[j] = sc;
      sel[j] = e < E ? sc + (bias != nullptr ? bias[e] : 0.0f) : NEG_INF;
    }
    if (topk_group < n_group) {
      const int gs = E / n_group;
      float my_group_score = NEG_INF;  // lane g holds the score of group g
      for (int g = 0; g < n_group; ++g) {
        float m1 = NEG_INF, m2 = NEG_INF;
        const int lo = g * gs, hi = lo + gs;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          const int e = j * 32 + lane;
          if (e >= lo && e < hi) {
            const float v = sel[j];
            if (value_above(v, m1)) { m2 = m1; m1 = v; } else if (value_above(v, m2)) { m2 = v; }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float b1 = __shfl_xor_sync(0xffffffffu, m1, o);
          const float b2 = __shfl_xor_sync(0xffffffffu, m2, o);
          const float n1 = max_nan_high(m1, b1);
          const float n2 = max_nan_high(min_nan_high(m1, b1), max_nan_high(m2, b2));
          m1 = n1;
          m2 = n2;
        }
        const float score = gs >= 2 ? m1 + m2 : m1;
        if (lane == g) my_group_score = score;
      }
      // top `topk_group` groups, ties to the lowest group index
      uint32_t group_mask = 0;
      bool taken = false;
      for (int r = 0; r < topk_group; ++r) {
        Cand c;
        c.v = (lane < n_group && !taken) ? my_group_score : NEG_INF;
        c.e = (lane < n_group && !taken) ? lane : 0x7fffffff;
        c.s = 0.f;
        c = warp_argmax(c);
        if (c.e < 32) {
          group_mask |= 1u << c.e;
          if (lane == c.e) taken = true;
        }
      }
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const int e = j * 32 + lane;
        if (e < E && !((group_mask >> (e / gs)) & 1u)) sel[j] = NEG_INF;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      sel[j] = x[j];
      pay[j] = x[j];
    }
    if (mode == 1) {
      // softmax_then_topk sorts probabilities.  A NaN, a +inf, or nothing but -inf in the row
      // makes every probability NaN, and a stable sort of equal keys keeps index order.
      float mx = NEG_INF;
      bool odd = false;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        if (j * 32 + lane < E) {
          odd = odd || (x[j] != x[j]);
          mx = fmaxf(mx, x[j]);
        }
      }
      mx = warp_max(mx);
      odd = __any_sync(0xffffffffu, odd) || mx == -NEG_INF || mx == NEG_INF;
      if (odd) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) sel[j] = __int_as_float(0x7fc00000);
      }
    }
  }

  // K rounds of warp arg-max over the not-yet-selected experts.
  uint32_t selected = 0;
  float my_val = 0.f;  // lane k keeps the payload of the k-th pick
  int my_id = 0;
  float first_pay = 0.f;
  for (int k = 0; k < K; ++k) {
    Cand c;
    c.v = NEG_INF;
    c.e = 0x7fffffff;
    c.s = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      if (e < E && !((selected >> j) & 1u) && better(sel[j], e, c.v, c.e)) {
        c.v = sel[j];
        c.e = e;
        c.s = pay[j];
      }
    }
    c = warp_argmax(c);
    if ((c.e & 31) == lane && c.e < E) selected |= 1u << (c.e >> 5);
    if (k == 0) first_pay = c.s;
    if (lane == k) {
      my_val = c.s;
      my_id = c.e;
    }
  }

  float w = 0.f;
  if (mode == 2) {
    float sum = 0.f;
    for (int k = 0; k < K; ++k) sum += __shfl_sync(0xffffffffu, my_val, k);
    w = __fdiv_rn(my_val, sum) * routed_scaling;
  } else if (mode == 1) {
    float mx = NEG_INF;
#pragma unroll
    for (int j = 0; j < EPL; ++j) mx = fmaxf(mx, x[j]);
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) sum += (j * 32 + lane < E) ? expf(x[j] - mx) : 0.f;
    sum = warp_sum(sum);
    w = __fdiv_rn(expf(my_val - mx), sum);
  } else {
    const float ex = lane < K ? expf(my_val - first_pay) : 0.f;
    float sum = 0.f;
    for (int k = 0; k < K; ++k) sum += __shfl_sync(0xffffffffu, ex, k);
    w = __fdiv_rn(ex, sum);
  }
  if (lane < K) {
    weights[(long long)t * K + lane] = w;
    ids[(long long)t * K + lane] = my_id;
  }
}

// ---------------------------------------------------------------------------
// sort_assignments
// ---------------------------------------------------------------------------
// An id outside [0, E) is reported in the status block and sorted as the nearest valid
// expert, so `order` and `slots` are always complete permutations: the kernels that index
// with them never see an unwritten entry.
__device__ __forceinline__ int clamp_id(int e, int E) { return e < 0 ? 0 : (e >= E ? E - 1 : e); }

__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const int* __restrict__ ids, int R, int E, int* __restrict__ chunk_hist, int* status) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += kSortThreads) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortChunk;
  for (int i = threadIdx.x; i < kSortChunk; i += kSortThreads) {
    const int idx = base + i;
    if (idx < R) {
      int e = ids[idx];
      if (e < 0 || e >= E) {
        report_error(status, ERR_BAD_OFFSETS, 10, idx);
        e = clamp_id(e, E);
      }
      atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kSortThreads) chunk_hist[(long long)blockIdx.x * E + e] = hist[e];
}

// One block of 1024 threads: per expert an exclusive scan over chunks (in place), then an
// exclusive scan over experts.
__global__ void __launch_bounds__(1024)
sort_scan_kernel(int* __restrict__ chunk_hist, int nchunks, int E, int R, int* __restrict__ offsets,
                 long long* __restrict__ counts64) {
  __shared__ int warp_tot[32];
  const int e = threadIdx.x;
  int total = 0;
  if (e < E) {
    for (int b = 0; b < nchunks; ++b) {
      const long long at = (long long)b * E + e;
      const int v = chunk_hist[at];
      chunk_hist[at] = total;
      total += v;
    }
    if (counts64 != nullptr) counts64[e] = total;
  }
  // block exclusive scan of `total`
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = total;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_tot[lane];
    int inc2 = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc2, o);
      if (lane >= o) inc2 += u;
    }
    warp_tot[lane] = inc2 - v;
  }
  __syncthreads();
  if (e < E) offsets[e] = warp_tot[warp] + incl - total;
  if (e == 0) offsets[E] = R;
}

__global__ void __launch_bounds__(kSortThreads)
sort_scatter_kernel(const int* __restrict__ ids, int R, int E, const int* __restrict__ chunk_base,
                    const int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ slots) {
  extern __shared__ int cnt[];  // [kSortWarps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kSortWarps * E; i += kSortThreads) cnt[i] = 0;
  __syncthreads();
  constexpr int kPerWarp = kSortChunk / kSortWarps;
  const int wbase = blockIdx.x * kSortChunk + warp * kPerWarp;
  int* mine = cnt + warp * E;
  for (int i = lane; i < kPerWarp; i += 32) {
    const int idx = wbase + i;
    if (idx < R) {
      atomicAdd(&mine[clamp_id(ids[idx], E)], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kSortThreads) {
    int base = offsets[e] + chunk_base[(long long)blockIdx.x * E + e];
    for (int w = 0; w < kSortWarps; ++w) {
      const int v = cnt[w * E + e];
      cnt[w * E + e] = base;
      base += v;
    }
  }
  __syncthreads();
  for (int i = lane; i < kPerWarp; i += 32) {
    const int idx = wbase + i;
    int e = -1;
    if (idx < R) e = clamp_id(ids[idx], E);
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int pos = 0;
    if (e >= 0) pos = mine[e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) mine[e] += __popc(peers);
    __syncwarp();
    if (e >= 0) {
      order[pos] = idx;
      slots[idx] = pos;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200moe_route_topk(const float* logits, long long ld, int tokens, int experts, int top_k,
                                  int mode, const float* bias, int n_group, int topk_group,
                                  float routed_scaling, float* weights, int32_t* ids, void* stream) {
  if (!logits || !weights || !ids) return B200MOE_ERR_ARG;
  if (tokens < 0 || experts <= 0 || top_k <= 0 || top_k > experts || mode < 0 || mode > 2)
    return B200MOE_ERR_ARG;
  if (experts > 1024 || top_k > 32) return B200MOE_ERR_LIMIT;
  if (mode == 2) {
    if (n_group <= 0 || topk_group <= 0 || experts % n_group != 0) return B200MOE_ERR_ARG;
    if (n_group > 32 && topk_group < n_group) return B200MOE_ERR_LIMIT;
  }
  if (tokens == 0) return B200MOE_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((tokens + kRouteWarps - 1) / kRouteWarps);
  const int epl = (experts + 31) / 32;
#define LAUNCH_ROUTE(EPL)                                                                              \
  route_topk_kernel<EPL><<<grid, kRouteWarps * 32, 0, s>>>(logits, ld, tokens, experts, top_k, mode,   \
                                                          bias, n_group, topk_group, routed_scaling,   \
                                                          weights, ids)
  if (epl <= 1) LAUNCH_ROUTE(1);
  else if (epl <= 2) LAUNCH_ROUTE(2);
  else if (epl <= 4) LAUNCH_ROUTE(4);
  else if (epl <= 8) LAUNCH_ROUTE(8);
  else if (epl <= 16) LAUNCH_ROUTE(16);
  else LAUNCH_ROUTE(32);
#undef LAUNCH_ROUTE
  return launch_status();
}

extern "C" long long b200moe_sort_assignments_workspace_bytes(long long assignments, int experts) {
  if (assignments < 0 || experts <= 0) return -1;
  const long long nchunks = (assignments + kSortChunk - 1) / kSortChunk;
  return (nchunks > 0 ? nchunks : 1) * (long long)experts * 4;
}

// The launches of the sort, shared by the entry point that takes a caller workspace and the
// one that uses the library's own static scratch.
static int launch_sort(const int32_t* ids, int R, int experts, int32_t* order, int32_t* offsets,
                       int32_t* slots, long long* counts64, int* chunk_hist, int32_t* status,
                       cudaStream_t s);

extern "C" int b200moe_sort_assignments(const int32_t* ids, long long assignments, int experts,
                                        int32_t* order, int32_t* offsets, int32_t* slots,
                                        long long* counts64, void* workspace, int32_t* status,
                                        void* stream) {
  if (!ids || !order || !offsets || !slots || !workspace || !status) return B200MOE_ERR_ARG;
  if (assignments < 0 || experts <= 0) return B200MOE_ERR_ARG;
  if (experts > 1024 || assignments > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  return launch_sort(ids, (int)assignments, experts, order, offsets, slots, counts64,
                     reinterpret_cast<int*>(workspace), status, reinterpret_cast<cudaStream_t>(stream));
}

static int launch_sort(const int32_t* ids, int R, int experts, int32_t* order, int32_t* offsets,
                       int32_t* slots, long long* counts64, int* chunk_hist, int32_t* status,
                       cudaStream_t s) {
  const int nchunks = (R + kSortChunk - 1) / kSortChunk;
  if (nchunks > 0) {
    sort_hist_kernel<<<nchunks, kSortThreads, experts * 4, s>>>(ids, R, experts, chunk_hist, status);
  }
  sort_scan_kernel<<<1, 1024, 0, s>>>(chunk_hist, nchunks, experts, R, offsets, counts64);
  if (nchunks > 0) {
    sort_scatter_kernel<<<nchunks, kSortThreads, kSortWarps * experts * 4, s>>>(ids, R, experts, chunk_hist,
                                                                              offsets, order, slots);
  }
  return launch_status();
}

// ---------------------------------------------------------------------------
// b200moe_sort_assignments_static: the same sort for callers that cannot obtain a workspace.
//
// Some hosts of this library have no allocator to offer: a serving process that handed all
// of HBM to its own arena at start-up, or a call site (a driver callback, a latency-critical
// loop) where cudaMalloc is off limits because it may synchronise the whole device.  For them
// the per-chunk histogram lives in a fixed 1 MiB array that is part of the library image, so
// this entry point allocates nothing and calls no allocating routine.  The price: every GPU
// that loads the library carries the array until the process exits, the problem size is
// capped (chunks * experts <= 262144 ints, chunks = ceil(assignments / 4096)), and all calls
// share the one array.  The array keeps whatever the previous call left in it; that is
// harmless because the histogram pass rewrites every entry the later passes read, so nothing
// has to start at zero.  Two calls whose kernels overlap on the GPU (different streams,
// several host threads) would race on the array: keep calls on one stream or order them.
//
// The array's device address is looked up on the first call made with a given device
// current (cudaGetSymbolAddress); make that first call outside any stream capture.
// ---------------------------------------------------------------------------
namespace b200 {
constexpr long long kStaticSortInts = 262144;  // 1 MiB
static __device__ __align__(256) int g_sort_scratch[kStaticSortInts];
}  // namespace b200

#include <mutex>

// In host code `g_sort_scratch` is only a handle for the symbol, not something a kernel can
// dereference; the device address is looked up once per device, with that device current.
static int static_sort_scratch(int** out) {
  static std::mutex lock;
  static int* address[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200MOE_ERR_ARG;
  std::lock_guard<std::mutex> guard(lock);
  if (address[dev] == nullptr) {
    int* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), b200::g_sort_scratch) != cudaSuccess ||
        ptr == nullptr)
      return B200MOE_ERR_DRIVER;
    address[dev] = ptr;
  }
  *out = address[dev];
  return B200MOE_OK;
}

extern "C" int b200moe_sort_assignments_static(const int32_t* ids, long long assignments, int experts,
                                               int32_t* order, int32_t* offsets, int32_t* slots,
                                               long long* counts64, int32_t* status, void* stream) {
  if (!ids || !order || !offsets || !slots || !status) return B200MOE_ERR_ARG;
  if (assignments < 0 || experts <= 0) return B200MOE_ERR_ARG;
  if (experts > 1024 || assignments > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  const long long nchunks = (assignments + kSortChunk - 1) / kSortChunk;
  if (nchunks * experts > kStaticSortInts) return B200MOE_ERR_LIMIT;
  int* scratch = nullptr;
  const int rc = static_sort_scratch(&scratch);
  if (rc != B200MOE_OK) return rc;
  return launch_sort(ids, (int)assignments, experts, order, offsets, slots, counts64, scratch, status,
                     reinterpret_cast<cudaStream_t>(stream));
}
