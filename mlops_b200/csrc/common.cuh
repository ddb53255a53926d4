// Device-side building blocks shared by the sm_100a kernels of this library:
// mbarrier helpers with bounded waits, TMA (cp.async.bulk.tensor) loads without
// cluster multicast, tcgen05 (UMMA / TMEM) wrappers and shared-memory matrix
// descriptors.  Everything here is inline PTX; nothing is taken from a library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ----------------------------------------------------------------------------
// Status word protocol.  Every kernel that can wait on something takes a device
// pointer to an int32[4] status block:
//   [0] first error code (0 = none), [1] block index, [2] where, [3] detail.
// A wait that runs out records where it gave up and the kernel unwinds; the
// host reads the block after a synchronisation of its own choosing.
// ----------------------------------------------------------------------------
enum : int {
  ERR_NONE = 0,
  ERR_WAIT_TIMEOUT = 1,   // an mbarrier wait ran past its limit
  ERR_BAD_OFFSETS = 2     // group offsets not monotone / out of range
};

__device__ __forceinline__ void report_error(int* status, int code, int where, int detail) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = where;
    status[3] = detail;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of the phase (try_wait may put the thread to sleep for a while; a role
// that sits on the critical path of a handshake polls with this instead).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Hardware (named) barriers of the CTA: ids 1..15, id 0 is __syncthreads.  `threads` is the
// total number of threads that take part in one completion (a multiple of 32); every thread of
// a participating warp must execute the instruction.  An arrival does not block.  Unlike an
// mbarrier these do not go through shared memory, whose queue is long while the tensor cores
// and the TMA unit stream operands through it.
__device__ __forceinline__ void named_arrive(uint32_t id, uint32_t threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- CTA pairs (thread-block clusters of two) -----------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of every CTA of the cluster arrives, then waits.  A hardware barrier: it
// cannot spin forever as long as every CTA reaches it, which bounded waits guarantee.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One arrival on the mbarrier at the same shared-memory offset in CTA `cta` of the cluster.
// This form orders the arrival after the thread's earlier accesses at CTA scope only: enough
// when what the waiter consumes was written by the async proxy (TMA) or sits in TMEM.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(smem_u32(bar)), "r"(cta)
      : "memory");
}

// The same arrival with release semantics at cluster scope: the waiter in the other CTA may
// consume what this thread (and, through the fence before it, its warp) wrote to shared memory
// with ordinary stores.  Costs about a microsecond; used only where such stores happened.
__device__ __forceinline__ void mbar_arrive_remote_release(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(smem_u32(bar)), "r"(cta)
      : "memory");
}

// Upper bound of any single wait, in SM clock cycles (about two seconds).
#ifndef B200_WAIT_LIMIT_CYCLES
#define B200_WAIT_LIMIT_CYCLES (4000000000LL)
#endif

// Bounded wait.  Returns false when the limit ran out or when another role of
// this CTA already raised the abort flag; the caller must then unwind.  try_wait itself
// suspends the thread for a hardware-defined time, so the abort flag and the clock are
// looked at only every few rounds.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where) {
  if (mbar_try(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t round = 1;; ++round) {
    if (mbar_try(bar, parity)) return true;
    if ((round & 7u) != 0) continue;
    if (*abort_flag) return false;
    if (clock64() - start > B200_WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      report_error(status, ERR_WAIT_TIMEOUT, where, (int)parity);
      return false;
    }
  }
}

// Bounded wait that polls without sleeping: for single threads whose wake-up latency is on
// the critical path (the UMMA issuers, lane 0 of an epilogue warp).
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where) {
  if (mbar_test(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t round = 1;; ++round) {
    if (mbar_test(bar, parity)) return true;
    if ((round & 63u) != 0) continue;
    if (*abort_flag) return false;
    if (clock64() - start > B200_WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      report_error(status, ERR_WAIT_TIMEOUT, where, (int)parity);
      return false;
    }
  }
}

// The same for a whole warp: lane 0 waits and tells the others, so a warp costs the barrier
// one poller instead of thirty-two.  The warp must be converged.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int where) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status, where) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// ... and with the non-sleeping poll, for waits that sit on a per-K-block handshake.  (A long
// wait should sleep: on a power-capped part a spinning lane costs clock frequency.)
__device__ __forceinline__ bool mbar_spin_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int where) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_spin(bar, parity, abort_flag, status, where) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ----------------------------------------------------------------------------
// TMA tiled loads (never multicast): global -> this CTA's shared memory,
// completion counted in bytes on an mbarrier.  The innermost coordinate times the
// element size must be a multiple of 16 bytes.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
// TMA tiled store: this CTA's shared memory -> global, tracked by the thread's bulk groups.
// The writes to shared memory must be made visible to the async proxy first
// (fence_proxy_async_smem by the writers, then a barrier among them and the issuing thread).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns when the thread's bulk stores have read their shared-memory source (it may be rewritten) ...
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... and when they are complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory management, MMA issue, commit, loads
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; E4M3/E5M2 operands, fp32 accumulate.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same for f16/bf16 operands.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival once every MMA issued before this point has retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_smem_addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_smem_addr)
               : "memory");
}
// ---- the same for a CTA pair (cta_group::2): allocation by one warp of EACH CTA, one MMA
// issued by the leader CTA spans both SMs, commits arrive on the barriers of both CTAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the mbarrier at this offset in every CTA named by `cta_mask`, once all MMAs
// issued so far have retired (a commit; it carries no load).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane
// (taddr.lane + i), columns taddr.col .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// ----------------------------------------------------------------------------
// Descriptors
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor of a 128-byte-swizzled operand tile (the layout a
// TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces; tile base 1024-byte aligned).
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1 (Blackwell)
//   bits [61,64) layout type, 2 = SWIZZLE_128B, 4 = SWIZZLE_64B
// K-major tile (rows of 128 bytes along K): stride offset = 8 rows = 1024 bytes.
// MN-major tile (rows of 128 bytes along M/N, one row per K index): stride offset =
// 8 K-rows = 1024 bytes, leading offset = distance between 128-byte-wide column panels.
// With SWIZZLE_64B the rows are 64 bytes (what a TMA load with CU_TENSOR_MAP_SWIZZLE_64B
// produces; tile base 512-byte aligned) and 8 of them are 512 bytes.
constexpr uint32_t kLayoutSwizzle128 = 2, kLayoutSwizzle64 = 4;
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes,
                                                            uint32_t layout = kLayoutSwizzle128) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout << 61;
  return d;
}

// Instruction descriptor (dense, fp32 accumulate):
//   [4,6) D format 1=f32   [7,10) A format   [10,13) B format
//   bit 15 A major (1 = MN-major)   bit 16 B major   [17,23) N>>3   [24,29) M>>4
// Formats: kind::f8f6f4 0 = E4M3, 1 = E5M2; kind::f16 0 = F16, 1 = BF16.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                  uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// RN-even conversion to E4M3 with saturation to +-448 (finite).
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

constexpr float kInv448 = 1.0f / 448.0f;

// E4M3 bytes of clamp(v / scale, +-448) with the division rounded to nearest, i.e. exactly
// what `x / scale` followed by the cast gives on a CPU.  Fast path: multiply by the rounded
// reciprocal; the true quotient lies within 2^-22 (relative) of that product, and the cast is
// monotonic, so when both ends of the interval [q(1-2^-21), q(1+2^-21)] cast to the same
// byte that byte is the exact answer.  Otherwise (a value within an ulp of an E4M3 rounding
// boundary, about one lane in ten thousand) the eight values take the exact division.
__device__ __forceinline__ uint2 quantize8(const float (&v)[8], float scale) {
  const float inv = __frcp_rn(scale);
  uint32_t w[2] = {0, 0};
  bool exact = true;
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    const float q0 = v[i] * inv, q1 = v[i + 1] * inv;
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
      float q = __fdiv_rn(v[i], scale);
      q = fminf(fmaxf(q, -448.0f), 448.0f);
      w[i >> 2] |= (uint32_t)to_e4m3(q) << (8 * (i & 3));
    }
  }
  return make_uint2(w[0], w[1]);
}

}  // namespace b200
