// Routing statistics and the routing VJP on the [tokens, experts] logits, one pass each.
//
// routing_probability_sum: column sums of the per-token probabilities (softmax of the logits,
// or sigmoid scores normalised per token), the `probability_sum` of the reference's
// `routing_statistics` (src/mlops/providers/moe_common.py:32-71).  The sum is formed in a fixed
// order (per-block partials over a contiguous token range, then a serial pass over the blocks),
// so it is bitwise repeatable.
//
// routing_gradient: the fp32 gradient of the logits from the cotangents of the route weights,
// of the auxiliary loss and of the probability sum, one warp per token
// (src/mlops/providers/moe_common.py:74-124, src/mlops/kernels/moe_router.py:403-502):
//   topk_then_softmax   d[id_k] = w_k (g_k - sum_k g_k w_k)
//   softmax_then_topk   d[e] = -p_e sum_k g_k p[id_k];  d[id_k] += g_k p[id_k]
//   sigmoid_noaux_tc    d[id_k] = ((sum_k w_k) g_k - sum_k g_k w_k) / (sum_k s[id_k]) * s[id_k] (1 - s[id_k])
//   auxiliary loss      softmax modes: d[e] += c p_e (f_e - p.f),  c = grad_aux * aux_scale
//                       sigmoid mode:  d[e] += c (f_e - p.f) s_e (1 - s_e),  c = grad_aux * aux_scale / sum_e s_e
//   probability sum     d[e] += j_e (gs_e - p.gs),  j_e = p_e (softmax modes) or (1 - s_e) p_e
// with lane l of the warp holding experts l, l + 32, ...
#include "common.cuh"
#include "host_util.h"

namespace b200 {

constexpr int kStatWarps = 8;

// p[j] (and, for the sigmoid mode, the raw scores s[j] and their row sum) of one logits row.
template <int EPL>
__device__ __forceinline__ void row_probabilities(const float* __restrict__ row, int E, int mode, int lane,
                                                  float (&p)[EPL], float (&s)[EPL], float& row_sum) {
  const float NEG_INF = __int_as_float(0xff800000);
  if (mode == 2) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      s[j] = e < E ? __fdiv_rn(1.0f, 1.0f + expf(-row[e])) : 0.f;
      sum += s[j];
    }
    row_sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < EPL; ++j) p[j] = __fdiv_rn(s[j], row_sum);
  } else {
    float x[EPL];
    float mx = NEG_INF;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      x[j] = e < E ? row[e] : NEG_INF;
      mx = fmaxf(mx, x[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      p[j] = (j * 32 + lane < E) ? expf(x[j] - mx) : 0.f;
      sum += p[j];
    }
    row_sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      p[j] = __fdiv_rn(p[j], row_sum);
      s[j] = p[j];
    }
  }
}

template <int EPL>
__global__ void __launch_bounds__(kStatWarps * 32)
probability_partials_kernel(const float* __restrict__ logits, long long ld, long long tokens, int E, int mode,
                            long long tokens_per_block, float* __restrict__ partials) {
  extern __shared__ float warp_sums[];  // [kStatWarps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long lo = (long long)blockIdx.x * tokens_per_block;
  const long long hi = min(lo + tokens_per_block, tokens);
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  for (long long t = lo + warp; t < hi; t += kStatWarps) {  // a fixed order per warp
    float p[EPL], s[EPL], row_sum;
    row_probabilities<EPL>(logits + t * ld, E, mode, lane, p, s, row_sum);
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc[j] += p[j];
  }
#pragma unroll
  for (int j = 0; j < EPL; ++j)
    if (j * 32 + lane < E) warp_sums[warp * E + j * 32 + lane] = acc[j];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kStatWarps * 32) {
    float v = 0.f;
    for (int w = 0; w < kStatWarps; ++w) v += warp_sums[w * E + e];  // warps in order
    partials[(long long)blockIdx.x * E + e] = v;
  }
}

__global__ void probability_finish_kernel(const float* __restrict__ partials, int blocks, int E,
                                          float* __restrict__ psum) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  float v = 0.f;
  for (int b = 0; b < blocks; ++b) v += partials[(long long)b * E + e];  // blocks in order
  psum[e] = v;
}

template <int EPL>
__global__ void __launch_bounds__(kStatWarps * 32)
routing_gradient_kernel(const float* __restrict__ logits, long long ld, long long tokens, int E, int K, int mode,
                        const int* __restrict__ ids, const float* __restrict__ weights,
                        const float* __restrict__ grad_weights, const float* __restrict__ grad_aux,
                        const float* __restrict__ frequency, float aux_scale,
                        const float* __restrict__ grad_psum, float* __restrict__ out, long long ldo) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kStatWarps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float p[EPL], s[EPL], d[EPL], row_sum;
  row_probabilities<EPL>(logits + t * ld, E, mode, lane, p, s, row_sum);
#pragma unroll
  for (int j = 0; j < EPL; ++j) d[j] = 0.f;

  // lane k < K holds the k-th pick of the token
  int id = -1;
  float w = 0.f, g = 0.f;
  if (lane < K) {
    id = ids[t * K + lane];
    if (id < 0 || id >= E) id = -1;  // (clamped and reported by the sort; contributes nothing here)
    w = weights != nullptr ? weights[t * K + lane] : 0.f;
    g = grad_weights[t * K + lane];
  }
  // value of the picked expert (its score for the sigmoid mode, its probability otherwise)
  float picked = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = __shfl_sync(0xffffffffu, id, k);
    float mine = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (j * 32 + lane == e) mine = s[j];
    const float v = __shfl_sync(0xffffffffu, mine, e < 0 ? 0 : (e & 31));
    if (lane == k) picked = e < 0 ? 0.f : v;
  }
  float contribution = 0.f;
  if (mode == 2) {
    const float picked_sum = warp_sum(picked);
    const float scaling = warp_sum(w);
    const float dot = warp_sum(g * w);
    contribution = __fdiv_rn(scaling * g - dot, picked_sum) * picked * (1.0f - picked);
  } else if (mode == 0) {
    const float dot = warp_sum(g * w);
    contribution = w * (g - dot);
  } else {
    const float dot = warp_sum(g * picked);
#pragma unroll
    for (int j = 0; j < EPL; ++j) d[j] = -p[j] * dot;
    contribution = g * picked;
  }
  for (int k = 0; k < K; ++k) {
    const int e = __shfl_sync(0xffffffffu, id, k);
    const float c = __shfl_sync(0xffffffffu, contribution, k);
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (j * 32 + lane == e) d[j] += c;
  }

  if (grad_aux != nullptr && frequency != nullptr) {
    float f[EPL], pf = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      f[j] = e < E ? frequency[e] : 0.f;
      pf += p[j] * f[j];
    }
    pf = warp_sum(pf);
    const float ga = *grad_aux * aux_scale;
    if (mode == 2) {
      const float c = __fdiv_rn(ga, row_sum);
#pragma unroll
      for (int j = 0; j < EPL; ++j) d[j] += c * (f[j] - pf) * s[j] * (1.0f - s[j]);
    } else {
#pragma unroll
      for (int j = 0; j < EPL; ++j) d[j] += ga * p[j] * (f[j] - pf);
    }
  }
  if (grad_psum != nullptr) {
    float gs[EPL], pg = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      gs[j] = e < E ? grad_psum[e] : 0.f;
      pg += p[j] * gs[j];
    }
    pg = warp_sum(pg);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float jac = mode == 2 ? (1.0f - s[j]) * p[j] : p[j];
      d[j] += jac * (gs[j] - pg);
    }
  }
  float* orow = out + t * ldo;
#pragma unroll
  for (int j = 0; j < EPL; ++j)
    if (j * 32 + lane < E) orow[j * 32 + lane] = d[j];
}

static long long stat_blocks(long long tokens) {
  const long long by_tokens = (tokens + kStatWarps - 1) / kStatWarps;
  const long long cap = 128;  // partial sums are added serially afterwards: enough blocks to fill HBM, no more
  return by_tokens < cap ? (by_tokens > 0 ? by_tokens : 1) : cap;
}

}  // namespace b200

using namespace b200;

#define B200_DISPATCH_EPL(experts, CALL)      \
  do {                                        \
    const int epl_ = ((experts) + 31) / 32;   \
    if (epl_ <= 1) { CALL(1); }               \
    else if (epl_ <= 2) { CALL(2); }          \
    else if (epl_ <= 4) { CALL(4); }          \
    else if (epl_ <= 8) { CALL(8); }          \
    else if (epl_ <= 16) { CALL(16); }        \
    else { CALL(32); }                        \
  } while (0)

extern "C" long long b200moe_routing_probability_sum_workspace_bytes(long long tokens, int experts) {
  if (tokens < 0 || experts <= 0) return -1;
  return stat_blocks(tokens) * (long long)experts * 4;
}

extern "C" int b200moe_routing_probability_sum(const float* logits, long long ld, long long tokens, int experts,
                                               int mode, void* workspace, float* probability_sum, void* stream) {
  if (!logits || !workspace || !probability_sum || tokens < 0 || experts <= 0 || mode < 0 || mode > 2)
    return B200MOE_ERR_ARG;
  if (experts > 1024) return B200MOE_ERR_LIMIT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long blocks = stat_blocks(tokens);
  const long long per_block = (tokens + blocks - 1) / blocks;
  float* partials = reinterpret_cast<float*>(workspace);
#define CALL_PARTIALS(EPL)                                                                                  \
  probability_partials_kernel<EPL><<<(unsigned)blocks, kStatWarps * 32, kStatWarps * experts * 4, s>>>(     \
      logits, ld, tokens, experts, mode, per_block, partials)
  B200_DISPATCH_EPL(experts, CALL_PARTIALS);
#undef CALL_PARTIALS
  probability_finish_kernel<<<(experts + 255) / 256, 256, 0, s>>>(partials, (int)blocks, experts, probability_sum);
  return launch_status();
}

extern "C" int b200moe_routing_gradient(const float* logits, long long ld, long long tokens, int experts, int top_k,
                                        int mode, const int32_t* ids, const float* route_weights,
                                        const float* grad_route_weights, const float* grad_aux,
                                        const float* frequency, float aux_scale, const float* grad_probability_sum,
                                        float* grad_logits, long long ldg, void* stream) {
  if (!logits || !ids || !grad_route_weights || !grad_logits || tokens < 0 || experts <= 0 || top_k <= 0 ||
      mode < 0 || mode > 2)
    return B200MOE_ERR_ARG;
  if (mode != 1 && !route_weights) return B200MOE_ERR_ARG;
  if (experts > 1024 || top_k > 32) return B200MOE_ERR_LIMIT;
  if (tokens == 0) return B200MOE_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((tokens + kStatWarps - 1) / kStatWarps);
#define CALL_GRADIENT(EPL)                                                                                 \
  routing_gradient_kernel<EPL><<<grid, kStatWarps * 32, 0, s>>>(logits, ld, tokens, experts, top_k, mode,  \
                                                               ids, route_weights, grad_route_weights,    \
                                                               grad_aux, frequency, aux_scale,            \
                                                               grad_probability_sum, grad_logits, ldg)
  B200_DISPATCH_EPL(experts, CALL_GRADIENT);
#undef CALL_GRADIENT
  return launch_status();
}
