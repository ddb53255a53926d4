// HBM-bound row kernels around the grouped GEMMs: E4M3 quantisation of activation rows
// (optionally gathered into expert order), SwiGLU fused with the quantisation of its
// result, the routed SwiGLU backward, and the 128x128 weight-block quantiser.
//
// Scale equations (bit-reproducible on a CPU):
//   activation rows / 1x128 blocks: scale = max(amax * fp32(1/448), 1e-12)
//        (reference: src/mlops/kernels/quack_moe/quantize_rows.py:34-41)
//   weight 128x128 blocks:          scale = max(amax / 448, 1e-12)   (RN division)
//        (reference: src/mlops/kernels/block_fp8.py:48-60)
//   value: q = e4m3_rn(clamp(x / scale, -448, 448)) with an RN fp32 division.
//
// One warp owns one row; every lane moves 16 bytes per access, so a warp reads 512
// contiguous bytes of bf16 and writes 256 contiguous bytes of E4M3 per step.  A 128-wide
// scale block is the business of one half warp (16 lanes x 8 values).
#include "common.cuh"
#include "host_util.h"

namespace b200 {

constexpr int kRowWarps = 8;

__device__ __forceinline__ float halfwarp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 pack8_bf16(const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

// mode 0: one scale per 128-column block.  mode 1: one scale per row (two passes).
__global__ void __launch_bounds__(kRowWarps * 32)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, long long src_rows,
                     const int* __restrict__ gather, int gather_div, long long rows, int D,
                     uint8_t* __restrict__ q, long long ldq, float* __restrict__ scales, long long s_row,
                     long long s_kb, int mode, __nv_bfloat16* __restrict__ copy, long long ldc, int* status) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= rows) return;
  long long src = gather != nullptr ? (long long)(gather[r] / gather_div) : r;
  if (src < 0 || src >= src_rows) {  // a bad index is reported and reads row 0, never out of bounds
    if (lane == 0) report_error(status, ERR_BAD_OFFSETS, 20, (int)r);
    src = 0;
  }
  const __nv_bfloat16* xr = x + src * ldx;
  uint8_t* qr = q + r * ldq;
  if (mode == 0) {
    // two 256-column steps per iteration: both loads are in flight before either is used
    for (int c0 = 0; c0 < D; c0 += 512) {
      const int ca = c0 + lane * 8, cb = ca + 256;
      uint4 raw_a = make_uint4(0, 0, 0, 0), raw_b = make_uint4(0, 0, 0, 0);
      if (ca < D) raw_a = *reinterpret_cast<const uint4*>(xr + ca);
      if (cb < D) raw_b = *reinterpret_cast<const uint4*>(xr + cb);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = h == 0 ? ca : cb;
        float v[8];
        unpack8(h == 0 ? raw_a : raw_b, v);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = halfwarp_max(amax);
        const float scale = fmaxf(amax * kInv448, 1e-12f);
        if (c < D) {
          *reinterpret_cast<uint2*>(qr + c) = quantize8(v, scale);
          if ((lane & 15) == 0) scales[r * s_row + (long long)(c >> 7) * s_kb] = scale;
          if (copy != nullptr) *reinterpret_cast<uint4*>(copy + r * ldc + c) = h == 0 ? raw_a : raw_b;
        }
      }
    }
  } else {
    float amax = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    const float scale = fmaxf(amax * kInv448, 1e-12f);
    for (int c = lane * 8; c < D; c += 256) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
      *reinterpret_cast<uint2*>(qr + c) = quantize8(v, scale);
    }
    if (lane == 0) scales[r * s_row] = scale;
  }
}

// The same quantisation, token-major: every token row is read and quantised ONCE and the
// result is written to each of the `fanout` output rows `slots[t * fanout + k]` (the
// expert-ordered rows of the token's assignments), instead of once per output row.  Same bytes
// and scales as quantize_rows_kernel with gather = order / fanout; 1/fanout of its arithmetic
// and source reads, so the pass is bound by its writes.  1x128 scales only.
__global__ void __launch_bounds__(kRowWarps * 32)
quantize_scatter_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, long long tokens,
                        const int* __restrict__ slots, int fanout, long long rows_out, int D,
                        uint8_t* __restrict__ q, long long ldq, float* __restrict__ scales,
                        long long s_row, long long s_kb, __nv_bfloat16* __restrict__ copy, long long ldc,
                        int* status) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  // lane k < fanout holds destination k; a slot outside the output is reported and skipped
  long long mine = -1;
  if (lane < fanout) {
    mine = slots[t * fanout + lane];
    if (mine < 0 || mine >= rows_out) {
      report_error(status, ERR_BAD_OFFSETS, 24, (int)t);
      mine = -1;
    }
  }
  const __nv_bfloat16* xr = x + t * ldx;
  for (int c0 = 0; c0 < D; c0 += 512) {
    const int ca = c0 + lane * 8, cb = ca + 256;
    uint4 raw_a = make_uint4(0, 0, 0, 0), raw_b = make_uint4(0, 0, 0, 0);
    if (ca < D) raw_a = *reinterpret_cast<const uint4*>(xr + ca);
    if (cb < D) raw_b = *reinterpret_cast<const uint4*>(xr + cb);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = h == 0 ? ca : cb;
      const uint4 raw = h == 0 ? raw_a : raw_b;
      float v[8];
      unpack8(raw, v);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = halfwarp_max(amax);
      const float scale = fmaxf(amax * kInv448, 1e-12f);
      const uint2 packed = quantize8(v, scale);
      for (int k = 0; k < fanout; ++k) {
        const long long dst = __shfl_sync(0xffffffffu, mine, k);
        if (dst < 0 || c >= D) continue;
        *reinterpret_cast<uint2*>(q + dst * ldq + c) = packed;
        if ((lane & 15) == 0) scales[dst * s_row + (long long)(c >> 7) * s_kb] = scale;
        if (copy != nullptr) *reinterpret_cast<uint4*>(copy + dst * ldc + c) = raw;
      }
    }
  }
}

// act = silu(gate) * up computed in fp32 from h13 = [gate | up] (each F wide), rounded
// once: to E4M3 with 1x128 scales (act_q / scales) and, when act_bf16 is given, to bf16.
// Optional GLM clamp: gate capped at `limit`, up clipped to [-limit, limit].
__global__ void __launch_bounds__(kRowWarps * 32)
swiglu_quant_kernel(const __nv_bfloat16* __restrict__ h13, long long ldh, long long rows, int F,
                    uint8_t* __restrict__ act_q, long long ldq, float* __restrict__ scales,
                    long long s_row, long long s_kb, __nv_bfloat16* __restrict__ act_bf16,
                    long long lda, float limit, int limited) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= rows) return;
  const __nv_bfloat16* hr = h13 + r * ldh;
  for (int c0 = 0; c0 < F; c0 += 256) {
    const int c = c0 + lane * 8;
    float g[8], u[8], a[8];
    uint4 rg = make_uint4(0, 0, 0, 0), ru = make_uint4(0, 0, 0, 0);
    if (c < F) {
      rg = *reinterpret_cast<const uint4*>(hr + c);
      ru = *reinterpret_cast<const uint4*>(hr + F + c);
    }
    unpack8(rg, g);
    unpack8(ru, u);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float gi = g[i], ui = u[i];
      if (limited) {
        gi = fminf(gi, limit);
        ui = fminf(fmaxf(ui, -limit), limit);
      }
      const float sig = __frcp_rn(1.0f + expf(-gi));
      a[i] = gi * sig * ui;
      amax = fmaxf(amax, fabsf(a[i]));
    }
    amax = halfwarp_max(amax);
    const float scale = fmaxf(amax * kInv448, 1e-12f);
    if (c < F) {
      if (act_q != nullptr) {
        *reinterpret_cast<uint2*>(act_q + r * ldq + c) = quantize8(a, scale);
        if ((lane & 15) == 0) scales[r * s_row + (long long)(c >> 7) * s_kb] = scale;
      }
      if (act_bf16 != nullptr) *reinterpret_cast<uint4*>(act_bf16 + r * lda + c) = pack8_bf16(a);
    }
  }
}

// Routed SwiGLU backward in one pass over h13 and r (= dy_row @ W2, before the route
// weight).  With score = route weight of the row:
//   dscore[row]  = <r, act>
//   g            = score * r
//   dgate        = g * up * (sig + silu * (1 - sig)),  dup = g * silu
//   grad_h13     = [dgate | dup]  -> E4M3 with 1x128 scales (and bf16 when asked)
//   act_scaled   = score * act    (bf16; operand of the down weight's gradient)
// (reference: src/mlops/kernels/quack_moe/swiglu_rows.py:100-199)
// gh_bf16 may alias h13 (the gradient written over the saved pre-activation): each thread reads
// the sixteen h13 values of an iteration before it stores the sixteen gradients to the same
// addresses, and no other thread touches them.
__global__ void __launch_bounds__(kRowWarps * 32)
dswiglu_routed_kernel(const __nv_bfloat16* h13, long long ldh,  // may be the same buffer as gh_bf16
                      const __nv_bfloat16* __restrict__ rmat, long long ldr,
                      const float* __restrict__ route_weights, long long n_weights,
                      const int* __restrict__ order, long long rows, int F, float* __restrict__ dscore,
                      uint8_t* __restrict__ gh_q, long long ldq, float* __restrict__ gh_scales,
                      long long s_row, long long s_kb, __nv_bfloat16* gh_bf16,
                      long long ldg, __nv_bfloat16* __restrict__ act_scaled, long long lda, float limit,
                      int limited, int* status) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= rows) return;
  long long which = order[r];
  if (which < 0 || which >= n_weights) {
    if (lane == 0) report_error(status, ERR_BAD_OFFSETS, 21, (int)r);
    which = 0;
  }
  const float score = route_weights[which];
  const __nv_bfloat16* hr = h13 + r * ldh;
  const __nv_bfloat16* rr = rmat + r * ldr;
  float dot = 0.f;
  for (int c0 = 0; c0 < F; c0 += 256) {
    const int c = c0 + lane * 8;
    float g[8], u[8], rv[8], dg[8], du[8], as[8];
    uint4 rg = make_uint4(0, 0, 0, 0), ru = rg, rx = rg;
    if (c < F) {
      rg = *reinterpret_cast<const uint4*>(hr + c);
      ru = *reinterpret_cast<const uint4*>(hr + F + c);
      rx = *reinterpret_cast<const uint4*>(rr + c);
    }
    unpack8(rg, g);
    unpack8(ru, u);
    unpack8(rx, rv);
    float amax_g = 0.f, amax_u = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float gi = g[i], ui = u[i];
      if (limited) {
        gi = fminf(gi, limit);
        ui = fminf(fmaxf(ui, -limit), limit);
      }
      const float sig = __frcp_rn(1.0f + expf(-gi));
      const float silu = gi * sig;
      const float act = silu * ui;
      dot = fmaf(rv[i], act, dot);
      const float go = score * rv[i];
      float dgi = go * ui * (sig + silu * (1.0f - sig));
      float dui = go * silu;
      if (limited) {
        if (!(g[i] <= limit)) dgi = 0.f;
        if (!(u[i] >= -limit && u[i] <= limit)) dui = 0.f;
      }
      dg[i] = dgi;
      du[i] = dui;
      as[i] = score * act;
      amax_g = fmaxf(amax_g, fabsf(dgi));
      amax_u = fmaxf(amax_u, fabsf(dui));
    }
    amax_g = halfwarp_max(amax_g);
    amax_u = halfwarp_max(amax_u);
    if (c < F) {
      if (gh_q != nullptr) {
        const float sg = fmaxf(amax_g * kInv448, 1e-12f);
        const float su = fmaxf(amax_u * kInv448, 1e-12f);
        *reinterpret_cast<uint2*>(gh_q + r * ldq + c) = quantize8(dg, sg);
        *reinterpret_cast<uint2*>(gh_q + r * ldq + F + c) = quantize8(du, su);
        if ((lane & 15) == 0) {
          gh_scales[r * s_row + (long long)(c >> 7) * s_kb] = sg;
          gh_scales[r * s_row + (long long)((F + c) >> 7) * s_kb] = su;
        }
      }
      if (gh_bf16 != nullptr) {
        *reinterpret_cast<uint4*>(gh_bf16 + r * ldg + c) = pack8_bf16(dg);
        *reinterpret_cast<uint4*>(gh_bf16 + r * ldg + F + c) = pack8_bf16(du);
      }
      if (act_scaled != nullptr) *reinterpret_cast<uint4*>(act_scaled + r * lda + c) = pack8_bf16(as);
    }
  }
  dot = warp_sum(dot);
  if (lane == 0 && dscore != nullptr) dscore[r] = dot;
}

// One CTA per 128x128 block of a [E, out, in] weight (bf16 or fp32 source).
template <typename SrcT>
__global__ void __launch_bounds__(256)
quantize_blocks_kernel(const SrcT* __restrict__ w, int out, int in, int blocks_out, int blocks_in,
                       uint8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float red[8];
  const long long e = blockIdx.z;
  const int br = blockIdx.y, bc = blockIdx.x;
  const SrcT* base = w + e * (long long)out * in;
  uint8_t* qbase = q + e * (long long)out * in;
  const int tr = threadIdx.x >> 5;  // 8 row groups
  const int tc = threadIdx.x & 31;  // 32 column groups of 4
  float amax = 0.f;
  for (int rr = tr; rr < 128; rr += 8) {
    const int row = br * 128 + rr;
    if (row >= out) break;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int col = bc * 128 + tc * 4 + k;
      if (col < in) amax = fmaxf(amax, fabsf((float)base[(long long)row * in + col]));
    }
  }
  amax = warp_max(amax);
  if (tc == 0) red[tr] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
  if (threadIdx.x == 0) scale[(e * blocks_out + br) * blocks_in + bc] = s;
  for (int rr = tr; rr < 128; rr += 8) {
    const int row = br * 128 + rr;
    if (row >= out) break;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int col = bc * 128 + tc * 4 + k;
      if (col < in) {
        float v = __fdiv_rn((float)base[(long long)row * in + col], s);
        v = fminf(fmaxf(v, -448.0f), 448.0f);
        qbase[(long long)row * in + col] = to_e4m3(v);
      }
    }
  }
}


// ---------------------------------------------------------------------------------------
// Column-scaled E4M3 for the FP8 weight gradient: the rows of a group (an expert's tokens)
// share one scale per COLUMN, scale = max(amax over the group's rows * fp32(1/448), 1e-12),
// the row quantiser's equations applied to a column (reference: the per-feature scales of
// src/mlops/kernels/quack_moe/quantize_transpose.py:126-133).  The output stays token-major:
// the weight-gradient GEMM reads both operands MN-major, so no transpose is ever stored.
// `offsets` holds segments * groups + 1 row boundaries; range i belongs to group i % groups.
// Pass 1: column maxima of every 256-row x 256-column piece, merged with atomicMax on the bit
// pattern (non-negative floats order like their bits).  Pass 2: maxima -> scales in place.
// Pass 3: the cast.
// ---------------------------------------------------------------------------------------
constexpr int kColRows = 256;  // rows per block: 8 warps x 32 rows

// The range (index into offsets) that holds row r; ranges may be empty.
__device__ __forceinline__ int range_of_row(const int* __restrict__ offsets, int ranges, int r) {
  int lo = 0, hi = ranges;  // invariant: offsets[lo] <= r < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= r) lo = mid;
    else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(256)
column_amax_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int rows, int width,
                   const int* __restrict__ offsets, int groups, int segments, unsigned int* __restrict__ amax_bits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.y * 256 + lane * 8;
  const int r0 = blockIdx.x * kColRows + warp * 32;
  if (c >= width || r0 >= rows) return;
  const int ranges = groups * segments;
  const int r_begin = max(r0, offsets[0]);                       // rows outside the table belong to no group
  const int r_end = min(min(r0 + 32, rows), offsets[ranges]);
  if (r_begin >= r_end) return;
  int range = range_of_row(offsets, ranges, r_begin);
  int range_end = offsets[range + 1];
  float m[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  auto flush = [&](int g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (m[i] > 0.f) atomicMax(amax_bits + (long long)g * width + c + i, __float_as_uint(m[i]));
      m[i] = 0.f;
    }
  };
  for (int r = r_begin; r < r_end; ++r) {
    if (r >= range_end) {  // the row belongs to a later range: hand in what this one gathered
      flush(range % groups);
      range = range_of_row(offsets, ranges, r);
      range_end = offsets[range + 1];
    }
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(x + (long long)r * ldx + c), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = fmaxf(m[i], fabsf(v[i]));  // a NaN never wins: the scale stays finite
  }
  flush(range % groups);
}

__global__ void __launch_bounds__(256)
column_scale_kernel(float* __restrict__ scales, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < n) scales[i] = fmaxf(scales[i] * kInv448, 1e-12f);  // the maxima arrive as fp32 bit patterns
}

__global__ void __launch_bounds__(256)
column_cast_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int rows, int width,
                   const int* __restrict__ offsets, int groups, int segments, const float* __restrict__ scales,
                   uint8_t* __restrict__ q, long long ldq) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.y * 256 + lane * 8;
  const int r0 = blockIdx.x * kColRows + warp * 32;
  if (c >= width || r0 >= rows) return;
  const int ranges = groups * segments;
  const int r_begin = max(r0, offsets[0]);
  const int r_end = min(min(r0 + 32, rows), offsets[ranges]);
  int range = -1, range_end = -1;
  float sc[8], inv[8];
  for (int r = r_begin; r < r_end; ++r) {
    if (r >= range_end) {
      range = range_of_row(offsets, ranges, r);
      range_end = offsets[range + 1];
      const float* sg = scales + (long long)(range % groups) * width + c;
      const float4 a = *reinterpret_cast<const float4*>(sg), b = *reinterpret_cast<const float4*>(sg + 4);
      sc[0] = a.x; sc[1] = a.y; sc[2] = a.z; sc[3] = a.w;
      sc[4] = b.x; sc[5] = b.y; sc[6] = b.z; sc[7] = b.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) inv[i] = __frcp_rn(sc[i]);
    }
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(x + (long long)r * ldx + c), v);
    // the same exact-division shortcut as quantize8, with one scale per value
    uint32_t w[2] = {0, 0};
    bool exact = true;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const float q0 = v[i] * inv[i], q1 = v[i + 1] * inv[i + 1];
      const float e0 = q0 * 4.76837158203125e-7f, e1 = q1 * 4.76837158203125e-7f;  // 2^-21
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q0 + e0, q1 + e1), __NV_SATFINITE, __NV_E4M3);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0 - e0, q1 - e1), __NV_SATFINITE, __NV_E4M3);
      exact = exact && (hi == lo);
      w[i >> 2] |= (hi & 0xffffu) << (8 * (i & 3));
    }
    if (!exact) {
      w[0] = w[1] = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float qv = __fdiv_rn(v[i], sc[i]);
        qv = fminf(fmaxf(qv, -448.0f), 448.0f);
        w[i >> 2] |= (uint32_t)to_e4m3(qv) << (8 * (i & 3));
      }
    }
    *reinterpret_cast<uint2*>(q + (long long)r * ldq + c) = make_uint2(w[0], w[1]);
  }
}

}  // namespace b200

using namespace b200;

static inline unsigned row_grid(long long rows) { return (unsigned)((rows + kRowWarps - 1) / kRowWarps); }

extern "C" int b200moe_quantize_rows(const void* x, long long ldx, long long src_rows, const int32_t* gather,
                                     int gather_div, long long rows, int width, void* q, long long ldq,
                                     float* scales, long long scale_row_stride, long long scale_block_stride,
                                     int mode, void* copy, long long ldc, int32_t* status, void* stream) {
  if (!x || !q || !scales || !status || rows < 0 || width <= 0 || (mode != 0 && mode != 1)) return B200MOE_ERR_ARG;
  if (rows > 0 && (src_rows <= 0 || (gather == nullptr && src_rows < rows))) return B200MOE_ERR_ARG;
  if (copy != nullptr && (mode != 0 || (ldc % 8) || ((uintptr_t)copy & 15))) return B200MOE_ERR_ARG;
  if (gather != nullptr && gather_div <= 0) return B200MOE_ERR_ARG;
  if ((width % 8) || (ldx % 8) || (ldq % 8) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7))
    return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  quantize_rows_kernel<<<row_grid(rows), kRowWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, src_rows, gather, gather_div > 0 ? gather_div : 1, rows,
      width, reinterpret_cast<uint8_t*>(q), ldq, scales, scale_row_stride, scale_block_stride, mode,
      reinterpret_cast<__nv_bfloat16*>(copy), ldc, status);
  return launch_status();
}

extern "C" int b200moe_quantize_rows_scatter(const void* x, long long ldx, long long tokens, const int32_t* slots,
                                             int fanout, long long rows_out, int width, void* q, long long ldq,
                                             float* scales, long long scale_row_stride,
                                             long long scale_block_stride, void* copy, long long ldc,
                                             int32_t* status, void* stream) {
  if (!x || !slots || !q || !scales || !status || tokens < 0 || rows_out < 0 || width <= 0) return B200MOE_ERR_ARG;
  if (fanout <= 0 || fanout > 32) return B200MOE_ERR_LIMIT;
  if (copy != nullptr && ((ldc % 8) || ((uintptr_t)copy & 15))) return B200MOE_ERR_ALIGN;
  if ((width % 8) || (ldx % 8) || (ldq % 8) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7))
    return B200MOE_ERR_ALIGN;
  if (tokens == 0) return B200MOE_OK;
  quantize_scatter_kernel<<<row_grid(tokens), kRowWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, tokens, slots, fanout, rows_out, width,
      reinterpret_cast<uint8_t*>(q), ldq, scales, scale_row_stride, scale_block_stride,
      reinterpret_cast<__nv_bfloat16*>(copy), ldc, status);
  return launch_status();
}

extern "C" int b200moe_swiglu_quantize(const void* h13, long long ldh, long long rows, int width,
                                       void* act_q, long long ldq, float* scales,
                                       long long scale_row_stride, long long scale_block_stride,
                                       void* act_bf16, long long lda, float limit, int limited,
                                       void* stream) {
  if (!h13 || rows < 0 || width <= 0 || (!act_q && !act_bf16) || (act_q && !scales)) return B200MOE_ERR_ARG;
  if ((width % 8) || (ldh % 8) || (ldq % 8) || (lda % 8) || ((uintptr_t)h13 & 15) || ((uintptr_t)act_q & 7) ||
      ((uintptr_t)act_bf16 & 15))
    return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  swiglu_quant_kernel<<<row_grid(rows), kRowWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(h13), ldh, rows, width, reinterpret_cast<uint8_t*>(act_q), ldq,
      scales, scale_row_stride, scale_block_stride, reinterpret_cast<__nv_bfloat16*>(act_bf16), lda, limit,
      limited);
  return launch_status();
}

extern "C" int b200moe_dswiglu_routed(const void* h13, long long ldh, const void* r, long long ldr,
                                      const float* route_weights, long long n_weights, const int32_t* order,
                                      long long rows, int width, float* dscore, void* grad_h13_q, long long ldq,
                                      float* grad_h13_scales, long long scale_row_stride,
                                      long long scale_block_stride, void* grad_h13_bf16, long long ldg,
                                      void* act_scaled, long long lda, float limit, int limited,
                                      int32_t* status, void* stream) {
  if (!h13 || !r || !route_weights || !order || !status || rows < 0 || width <= 0) return B200MOE_ERR_ARG;
  if (rows > 0 && n_weights <= 0) return B200MOE_ERR_ARG;
  if (grad_h13_q && !grad_h13_scales) return B200MOE_ERR_ARG;
  if ((width % 8) || (ldh % 8) || (ldr % 8) || (ldq % 8) || (ldg % 8) || (lda % 8)) return B200MOE_ERR_ALIGN;
  if (((uintptr_t)h13 & 15) || ((uintptr_t)r & 15) || ((uintptr_t)grad_h13_q & 7) ||
      ((uintptr_t)grad_h13_bf16 & 15) || ((uintptr_t)act_scaled & 15))
    return B200MOE_ERR_ALIGN;
  if (rows == 0) return B200MOE_OK;
  dswiglu_routed_kernel<<<row_grid(rows), kRowWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(h13), ldh, reinterpret_cast<const __nv_bfloat16*>(r), ldr,
      route_weights, n_weights, order, rows, width, dscore, reinterpret_cast<uint8_t*>(grad_h13_q), ldq,
      grad_h13_scales, scale_row_stride, scale_block_stride, reinterpret_cast<__nv_bfloat16*>(grad_h13_bf16), ldg,
      reinterpret_cast<__nv_bfloat16*>(act_scaled), lda, limit, limited, status);
  return launch_status();
}

// E4M3 rows of x [rows, width] with one scale per (group, column): scales [groups, width].
// Rows outside every range (none, when offsets[0] == 0 and the last entry == rows) are not written.
extern "C" int b200moe_quantize_columns(const void* x, long long ldx, long long rows, int width,
                                        const int32_t* offsets, int groups, int segments, void* q, long long ldq,
                                        float* scales, void* stream) {
  if (!x || !offsets || !q || !scales || rows < 0 || width <= 0 || groups <= 0 || segments <= 0)
    return B200MOE_ERR_ARG;
  if (rows > 0x7fffffffLL) return B200MOE_ERR_LIMIT;
  if ((width % 8) || (ldx % 8) || (ldq % 8) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7) || ((uintptr_t)scales & 15))
    return B200MOE_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long n = (long long)groups * width;
  if (cudaMemsetAsync(scales, 0, (size_t)n * sizeof(float), s) != cudaSuccess) return B200MOE_ERR_LAUNCH;
  if (rows > 0) {
    dim3 grid((unsigned)((rows + kColRows - 1) / kColRows), (unsigned)((width + 255) / 256));
    column_amax_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, (int)rows, width,
                                            offsets, groups, segments, reinterpret_cast<unsigned int*>(scales));
  }
  column_scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(scales, n);
  if (rows > 0) {
    dim3 grid((unsigned)((rows + kColRows - 1) / kColRows), (unsigned)((width + 255) / 256));
    column_cast_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, (int)rows, width,
                                            offsets, groups, segments, scales, reinterpret_cast<uint8_t*>(q), ldq);
  }
  return launch_status();
}


extern "C" int b200moe_quantize_blocks(const void* w, int src_is_fp32, int experts, int out, int in,
                                       void* q, float* scale, void* stream) {
  if (!w || !q || !scale || experts <= 0 || out <= 0 || in <= 0) return B200MOE_ERR_ARG;
  if (experts > 65535) return B200MOE_ERR_LIMIT;
  const int bo = (out + 127) / 128, bi = (in + 127) / 128;
  if (bo > 65535) return B200MOE_ERR_LIMIT;
  dim3 grid(bi, bo, experts);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (src_is_fp32)
    quantize_blocks_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<const float*>(w), out, in, bo, bi,
                                                      reinterpret_cast<uint8_t*>(q), scale);
  else
    quantize_blocks_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(w), out,
                                                              in, bo, bi, reinterpret_cast<uint8_t*>(q), scale);
  return launch_status();
}
