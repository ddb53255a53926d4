// Un-permute / combine: out[t] = residual[t] + sum_k w[t,k] * src[slots[t,k]] in fp32,
// slots visited in the fixed order k = 0..K-1 and the sum rounded once, so the result
// is bitwise repeatable (reference: src/mlops/kernels/moe_dispatch.py:21-72, used by
// `combine` :168 and, without weights and residual, by `dispatch_backward` :136).
#include "common.cuh"
#include "host_util.h"

#include <stdlib.h>

namespace b200 {

constexpr int kCombineThreads = 128;

__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const __nv_bfloat16* __restrict__ src, long long lds, long long src_rows,
               const int* __restrict__ slots, const float* __restrict__ weights,
               const __nv_bfloat16* __restrict__ residual, long long ldr, __nv_bfloat16* __restrict__ out,
               long long ldo, int D, int K) {
  const long long t = blockIdx.x;
  const int* st = slots + t * K;
  const float* wt = weights != nullptr ? weights + t * K : nullptr;
  for (int c = threadIdx.x * 8; c < D; c += kCombineThreads * 8) {
    float acc[8];
    if (residual != nullptr) {
      const uint4 raw = *reinterpret_cast<const uint4*>(residual + t * ldr + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] = f.x;
        acc[2 * i + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      long long slot = st[k];
      if (slot < 0) continue;  // "no row here": a token copy whose assignment lives on another rank
      slot = slot >= src_rows ? src_rows - 1 : slot;
      const float w = wt != nullptr ? wt[k] : 1.0f;
      const uint4 raw = *reinterpret_cast<const uint4*>(src + slot * lds + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] = fmaf(f.x, w, acc[2 * i]);
        acc[2 * i + 1] = fmaf(f.y, w, acc[2 * i + 1]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * ldo + c) = o;
  }
}

// dst[r] = src[gather[r] / gather_div] (bf16 rows), the expert-ordered copy of token rows.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds, long long src_rows,
                   const int* __restrict__ gather, int gather_div, long long rows, int D,
                   __nv_bfloat16* __restrict__ dst, long long ldd, int* status) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  long long s = gather[r] / gather_div;
  if (s < 0 || s >= src_rows) {  // reported, and row 0 is copied instead of a read out of bounds
    if (lane == 0) report_error(status, ERR_BAD_OFFSETS, 22, (int)r);
    s = 0;
  }
  for (int c = lane * 8; c < D; c += 256)
    *reinterpret_cast<uint4*>(dst + r * ldd + c) = *reinterpret_cast<const uint4*>(src + s * lds + c);
}

// The dispatch of an expert-parallel layer as ONE kernel: gather + transfer.  Send row i is the
// bf16 row src[gather[i]]; the send rows are grouped by destination rank (send_start), and row i
// of the group for rank r is written straight into r's receive arena over NVLink (plain 16-byte
// stores through a peer mapping of that GPU's memory: no send buffer, no copy engine, no
// library collective).  Nothing in here waits for another GPU: the ranks meet afterwards, on the
// host side's collective, before anyone reads its arena.
constexpr int kPeerMaxRanks = 16;
struct PeerDispatchParams {
  __nv_bfloat16* dest[kPeerMaxRanks];  // base of every rank's arena slot, as mapped on THIS GPU
  int send_start[kPeerMaxRanks + 1];   // send rows [send_start[r], send_start[r+1]) go to rank r
  long long dest_row0[kPeerMaxRanks];  // first arena row at rank r that belongs to this sender
  long long dest_rows;                 // rows of an arena slot (bound of every destination row)
  int world;
};

constexpr int kPeerWarps = 16;  // rows in flight per CTA
__global__ void __launch_bounds__(kPeerWarps * 32)
peer_dispatch_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds, long long src_rows,
                          const int* __restrict__ gather, long long rows, int D, long long ldd,
                          const PeerDispatchParams pp, int* status) {
  const int lane = threadIdx.x & 31;
  // a few resident CTAs walk all rows (like a collective's kernel, this one runs beside the GEMMs
  // of the previous chunk and must leave them their SMs)
  for (long long i = (long long)blockIdx.x * kPeerWarps + (threadIdx.x >> 5); i < rows;
       i += (long long)gridDim.x * kPeerWarps) {
    int r = 0;
    while (r + 1 < pp.world && i >= pp.send_start[r + 1]) ++r;
    const long long s = gather[i];
    const long long d = pp.dest_row0[r] + (i - pp.send_start[r]);
    if (s < 0 || s >= src_rows || d < 0 || d >= pp.dest_rows) {  // reported; nothing is read or written out of bounds
      if (lane == 0) report_error(status, ERR_BAD_OFFSETS, 26, (int)i);
      continue;
    }
    __nv_bfloat16* dst = pp.dest[r] + d * ldd;
    const __nv_bfloat16* from = src + s * lds;
    int c = lane * 8;
    for (; c + 768 < D; c += 1024) {  // four 16-byte loads in flight per lane
      const uint4 v0 = *reinterpret_cast<const uint4*>(from + c), v1 = *reinterpret_cast<const uint4*>(from + c + 256);
      const uint4 v2 = *reinterpret_cast<const uint4*>(from + c + 512), v3 = *reinterpret_cast<const uint4*>(from + c + 768);
      *reinterpret_cast<uint4*>(dst + c) = v0;
      *reinterpret_cast<uint4*>(dst + c + 256) = v1;
      *reinterpret_cast<uint4*>(dst + c + 512) = v2;
      *reinterpret_cast<uint4*>(dst + c + 768) = v3;
    }
    for (; c < D; c += 256) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(from + c);
  }
}

// The sender's plan of a de-duplicated expert-parallel dispatch in one launch.  One copy of a token
// per rank that holds at least one of its K experts (rank = key / local), ordered by rank, then
// token.  Block r scans the tokens for rank r (copy_start[r] is where its copies begin) and writes
// for each copy: its token, and the metadata row [K local expert ids (-1: that assignment lives on
// another rank) | K route weights (fp32 bits; 0 for those)]; and for every (token, rank) the copy's
// position or -1.
struct CopyPlanParams {
  int copy_start[kPeerMaxRanks * 8 + 1];  // up to 128 ranks
};
__global__ void __launch_bounds__(1024)
build_copies_kernel(const int* __restrict__ keys, const float* __restrict__ weights, int tokens, int K, int world,
                    int local, const CopyPlanParams cp, int* __restrict__ token_of, int* __restrict__ meta,
                    int* __restrict__ token_copies, int* status) {
  __shared__ int warp_sums[32];
  __shared__ int running_s;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) running_s = cp.copy_start[r];
  __syncthreads();
  for (int base = 0; base < tokens; base += 1024) {
    const int t = base + tid;
    int has = 0;
    if (t < tokens) {
      for (int k = 0; k < K; ++k) {
        const int key = keys[(long long)t * K + k];
        has |= (key >= 0 && key / local == r) ? 1 : 0;
      }
    }
    // exclusive scan of `has` over the block
    int incl = has;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += v;
      }
      warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = running_s + (warp ? warp_sums[warp - 1] : 0) + incl - has;
    const int block_total = warp_sums[31];
    if (t < tokens) {
      if (has && before < cp.copy_start[r + 1]) {
        token_of[before] = t;
        for (int k = 0; k < K; ++k) {
          const int key = keys[(long long)t * K + k];
          const bool here = key >= 0 && key / local == r;
          meta[(long long)before * 2 * K + k] = here ? key - r * local : -1;
          meta[(long long)before * 2 * K + K + k] = here ? __float_as_int(weights[(long long)t * K + k]) : 0;
        }
        token_copies[(long long)t * world + r] = before;
      } else {
        token_copies[(long long)t * world + r] = -1;
      }
    }
    __syncthreads();
    if (tid == 0) running_s += block_total;
    __syncthreads();
  }
  if (tid == 0 && running_s != cp.copy_start[r + 1]) report_error(status, ERR_BAD_OFFSETS, 27, r);  // plan and keys disagree
}

// out[t, k] = values[slots[t, k]]: a per-sorted-row scalar brought back to assignment order.
__global__ void gather_scalar_kernel(const float* __restrict__ values, long long n_values,
                                     const int* __restrict__ slots, long long n, float* __restrict__ out,
                                     int* status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  long long s = slots[i];
  if (s < 0 || s >= n_values) {
    report_error(status, ERR_BAD_OFFSETS, 23, (int)i);
    s = 0;
  }
  out[i] = values[s];
}

// out[t] = bf16(sums[t] + residual[t]): the rounding that ends a combine whose route-weighted
// sum was formed in fp32 by the down projection's fused store.
__global__ void __launch_bounds__(256)
finish_combine_kernel(const float* __restrict__ sums, long long lds, const __nv_bfloat16* __restrict__ residual,
                      long long ldr, __nv_bfloat16* __restrict__ out, long long ldo, long long tokens, int D) {
  const int per_row = D / 8;
  const long long total = tokens * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    const float4 lo = *reinterpret_cast<const float4*>(sums + t * lds + c);
    const float4 hi = *reinterpret_cast<const float4*>(sums + t * lds + c + 4);
    float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    if (residual != nullptr) {
      const uint4 raw = *reinterpret_cast<const uint4*>(residual + t * ldr + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        v[2 * k] += f.x;
        v[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(out + t * ldo + c) = o;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200moe_combine(const void* src, long long lds, long long src_rows, const int32_t* slots,
                               const float* weights, const void* residual, long long ldr, void* out,
                               long long ldo, long long tokens, int width, int top_k, void* stream) {
  if (!src || !slots || !out || tokens < 0 || width <= 0 || top_k <= 0 || src_rows <= 0)
    return B200MOE_ERR_ARG;
  if ((width % 8) || (lds % 8) || (ldo % 8) || (residual && (ldr % 8))) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)src & 15) || ((uintptr_t)out & 15) || ((uintptr_t)residual & 15)) return B200MOE_ERR_ALIGN;
  if (tokens > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if (tokens == 0) return B200MOE_OK;
  combine_kernel<<<(unsigned)tokens, kCombineThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), lds, src_rows, slots, weights,
      reinterpret_cast<const __nv_bfloat16*>(residual), ldr, reinterpret_cast<__nv_bfloat16*>(out), ldo, width,
      top_k);
  return launch_status();
}

extern "C" int b200moe_gather_rows(const void* src, long long lds, long long src_rows, const int32_t* gather,
                                   int gather_div, long long rows, int width, void* dst, long long ldd,
                                   int32_t* status, void* stream) {
  if (!src || !gather || !dst || !status || rows < 0 || width <= 0 || gather_div <= 0) return B200MOE_ERR_ARG;
  if (rows > 0 && src_rows <= 0) return B200MOE_ERR_ARG;
  if ((width % 8) || (lds % 8) || (ldd % 8) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15))
    return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  gather_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), lds, src_rows, gather, gather_div, rows, width,
      reinterpret_cast<__nv_bfloat16*>(dst), ldd, status);
  return launch_status();
}

// Fused gather + transfer of an expert-parallel dispatch (see peer_dispatch_rows_kernel).
// `dest[r]`: the arena slot of rank r as mapped into this process (r == own rank: the local
// arena); `send_start` has world + 1 entries; `dest_row0[r]`: where this sender's rows start in
// r's slot; every destination row is bounded by `dest_rows`.  All pointers are bf16 rows of
// `width` elements with pitch `ldd` (destination) / `lds` (source).
extern "C" int b200moe_peer_dispatch_rows(const void* src, long long lds, long long src_rows,
                                          const int32_t* gather, long long rows, int width,
                                          void* const* dest, long long ldd, long long dest_rows,
                                          const int32_t* send_start, const long long* dest_row0, int world,
                                          int32_t* status, void* stream) {
  if (!src || !gather || !dest || !send_start || !dest_row0 || !status || rows < 0 || width <= 0 || world <= 0)
    return B200MOE_ERR_ARG;
  if (world > kPeerMaxRanks) return B200MOE_ERR_LIMIT;
  if ((width % 8) || (lds % 8) || (ldd % 8) || ((uintptr_t)src & 15)) return B200MOE_ERR_ALIGN;
  PeerDispatchParams pp;
  for (int r = 0; r < kPeerMaxRanks; ++r) {
    pp.dest[r] = r < world ? reinterpret_cast<__nv_bfloat16*>(dest[r]) : nullptr;
    pp.dest_row0[r] = r < world ? dest_row0[r] : 0;
    if (r < world && (!dest[r] || ((uintptr_t)dest[r] & 15))) return B200MOE_ERR_ALIGN;
  }
  for (int r = 0; r <= kPeerMaxRanks; ++r) pp.send_start[r] = send_start[r < world ? r : world];
  if (pp.send_start[0] != 0 || pp.send_start[world] != rows) return B200MOE_ERR_ARG;
  for (int r = 0; r < world; ++r)
    if (pp.send_start[r + 1] < pp.send_start[r]) return B200MOE_ERR_ARG;
  pp.dest_rows = dest_rows;
  pp.world = world;
  if (rows == 0) return B200MOE_OK;
  // at most `B200MOE_PEER_CTAS` CTAs (default 64) so the kernel can run beside the expert GEMMs
  static const int cta_cap = [] {
    const char* v = getenv("B200MOE_PEER_CTAS");
    const int n = v ? atoi(v) : 64;
    return n > 0 ? n : 64;
  }();
  long long blocks = (rows + kPeerWarps - 1) / kPeerWarps;
  if (blocks > cta_cap) blocks = cta_cap;
  peer_dispatch_rows_kernel<<<(unsigned)blocks, kPeerWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), lds, src_rows, gather, rows, width, ldd, pp, status);
  return launch_status();
}

// The sender's plan of a de-duplicated dispatch (see build_copies_kernel).  `copy_start` (host,
// world + 1 entries): where each rank's copies begin; copy_start[world] copies in all.
extern "C" int b200moe_build_copies(const int32_t* keys, const float* weights, int tokens, int top_k, int world,
                                    int local, const int32_t* copy_start, int32_t* token_of, int32_t* meta,
                                    int32_t* token_copies, int32_t* status, void* stream) {
  if (!keys || !weights || !copy_start || !token_of || !meta || !token_copies || !status) return B200MOE_ERR_ARG;
  if (tokens < 0 || top_k <= 0 || world <= 0 || local <= 0) return B200MOE_ERR_ARG;
  if (world > kPeerMaxRanks * 8) return B200MOE_ERR_LIMIT;
  CopyPlanParams cp;
  for (int r = 0; r <= kPeerMaxRanks * 8; ++r) cp.copy_start[r] = copy_start[r < world ? r : world];
  if (tokens == 0) return B200MOE_OK;
  build_copies_kernel<<<(unsigned)world, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      keys, weights, tokens, top_k, world, local, cp, token_of, meta, token_copies, status);
  return launch_status();
}

extern "C" int b200moe_gather_scalar(const float* values, long long n_values, const int32_t* slots, long long n,
                                     float* out, int32_t* status, void* stream) {
  if (!values || !slots || !out || !status || n < 0 || (n > 0 && n_values <= 0)) return B200MOE_ERR_ARG;
  if (n == 0) return B200MOE_OK;
  gather_scalar_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      values, n_values, slots, n, out, status);
  return launch_status();
}

extern "C" int b200moe_finish_combine(const float* sums, long long lds, const void* residual, long long ldr,
                                      void* out, long long ldo, long long tokens, int width, void* stream) {
  if (!sums || !out || tokens < 0 || width <= 0) return B200MOE_ERR_ARG;
  if ((width % 8) || (lds % 4) || (ldo % 8) || (residual && (ldr % 8))) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)sums & 15) || ((uintptr_t)out & 15) || ((uintptr_t)residual & 15)) return B200MOE_ERR_ALIGN;
  if (tokens == 0) return B200MOE_OK;
  const long long work = tokens * (width / 8);
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count_device() * 8;
  if (blocks > cap) blocks = cap;
  finish_combine_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sums, lds, reinterpret_cast<const __nv_bfloat16*>(residual), ldr, reinterpret_cast<__nv_bfloat16*>(out), ldo,
      tokens, width);
  return launch_status();
}
