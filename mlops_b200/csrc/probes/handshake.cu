// Stand-alone probe of the tensor-core hand-back loop the FP8 grouped GEMM is built on: how fast
// tcgen05.mma issues and retires, how long a commit takes to reach a waiting warp, and what the
// issue -> retire -> drain -> release -> re-issue ring of accumulator slabs sustains with no
// operand traffic at all (operands resident in shared memory, all zero).  Build and run:
//
//     python -m mlops_b200.probes handshake
//
// One CTA per SM, 13 warps (the GEMM has 12; the thirteenth is the stand-in producer of the
// four-issuer layout).  Every wait is bounded; the hardware (named) barriers
// are always arrived on, whatever the waits return.
#include "../common.cuh"

#include <cstdio>
using namespace b200;

__device__ __forceinline__ bool spin(uint64_t* bar, uint32_t parity) {
  for (long long i = 0; i < 100000000LL; ++i)
    if (mbar_test(bar, parity)) return true;
  return false;
}

__device__ __forceinline__ void issue_slab(uint32_t tmem, int j, uint64_t adesc, uint64_t bdesc, uint64_t* bar) {
  constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, 128, 128);
  const uint32_t d = tmem + j * 128;
  tc_fence_after_sync();
  umma_f8(d, adesc, bdesc, idesc, 0u);
  umma_f8(d, adesc + 2, bdesc + 2, idesc, 1u);
  umma_f8(d, adesc + 4, bdesc + 4, idesc, 1u);
  umma_f8(d, adesc + 6, bdesc + 6, idesc, 1u);
  umma_commit(bar);
}

// mode 0: issue rate, `count` K blocks of 128 x 256 x 128 back to back (narrow: as two N = 128 halves)
// mode 1: latency, `count` N = 128 multiplications + commit until a polling thread sees the barrier
// mode 2: the ring.  layout 0: two issuer warps x two slabs (the GEMM's); 1: four issuers x one
//         slab; 2: one issuer x four slabs.  epilogue 0: empty, 1: reads the slab, 2: reads + 128 FMAs.
//         features (layout 0): bit 0 a ring of four operand stages with full/empty barriers and a
//         stand-in producer, bit 1 the issuers read an abort flag every K block, bit 2 the epilogue
//         fetches two scales per K block from global memory four K blocks ahead
__global__ void __launch_bounds__(416, 1)
probe(int mode, int count, int narrow, int layout, int epilogue, int features, const float* scales, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar[4];
  __shared__ uint64_t full[4], empty[4];  // features bit 0: a ring of four operand stages
  __shared__ uint64_t fin;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], layout == 1 ? 2 : 1);  // one commit per issuer of the K block
    }
    abort_flag = 0;
    mbar_init(&fin, 1);
    fence_mbar_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(&slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t adesc = make_smem_desc(smem_u32(smem), 16, 1024);
  const uint64_t bdesc = make_smem_desc(smem_u32(smem + 16384), 16, 1024);

  if (mode == 0 && warp == 1 && lane == 0) {
    constexpr uint32_t idesc256 = make_idesc(0, 0, 0, 0, 128, 256);
    constexpr uint32_t idesc128 = make_idesc(0, 0, 0, 0, 128, 128);
    const long long t0 = clock64();
    for (int it = 0; it < count; ++it) {
      const uint32_t d = tmem + (it & 1) * 256;
      if (!narrow) {
        umma_f8(d, adesc, bdesc, idesc256, 0u);
        umma_f8(d, adesc + 2, bdesc + 2, idesc256, 1u);
        umma_f8(d, adesc + 4, bdesc + 4, idesc256, 1u);
        umma_f8(d, adesc + 6, bdesc + 6, idesc256, 1u);
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint64_t b = bdesc + (uint64_t)((h * 128 * 128) >> 4);
          umma_f8(d + h * 128, adesc, b, idesc128, 0u);
          umma_f8(d + h * 128, adesc + 2, b + 2, idesc128, 1u);
          umma_f8(d + h * 128, adesc + 4, b + 4, idesc128, 1u);
          umma_f8(d + h * 128, adesc + 6, b + 6, idesc128, 1u);
        }
      }
    }
    umma_commit(&fin);
    spin(&fin, 0);
    if (blockIdx.x == 0) out[0] = (clock64() - t0) / count;
  }
  if (mode == 1 && warp == 1 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, 128, 128);
    long long total = 0;
    for (int rep = 0; rep < 64; ++rep) {
      const long long t0 = clock64();
      for (int i = 0; i < count; ++i) umma_f8(tmem, adesc + 2 * (i & 3), bdesc + 2 * (i & 3), idesc, i ? 1u : 0u);
      umma_commit(&bar[0]);
      spin(&bar[0], rep & 1);
      total += clock64() - t0;
    }
    if (blockIdx.x == 0) out[0] = total / 64;
  }
  if (mode == 2) {
    const int pairs = count / 2;  // every slab is used once per pair of K blocks
    const bool staged = (features & 1) && layout <= 1;
    int first = -1, slabs = 0;
    if (layout == 0 && warp < 2) { first = 2 * warp; slabs = 2; }
    if (layout == 1 && warp < 4) { first = warp; slabs = 1; }
    if (layout == 2 && warp == 0) { first = 0; slabs = 4; }
    if (first >= 0) {
      const long long t0 = clock64();
      for (int u = 0; u < pairs; ++u) {
        const int it = 2 * u + (layout == 0 ? warp : warp >> 1);  // the K block of this warp's slab(s)
        if (staged) {
          int seen = 1;
          if (lane == 0) seen = spin(&full[it & 3], (it >> 2) & 1) ? 1 : 0;
          if (__shfl_sync(0xffffffffu, seen, 0) == 0) break;
        }
        for (int c = 0; c < slabs; ++c) {
          const int j = first + c;
          if (u >= 1) named_sync(1 + j, 160);  // the slab's four epilogue warps handed it back
          if (lane == 0) {
            issue_slab(tmem, j, adesc, bdesc, &bar[j]);
            if (staged && c == slabs - 1) umma_commit(&empty[it & 3]);
          }
          __syncwarp();
        }
        if (features & 2) {
          int aborted = lane == 0 ? *(volatile int*)&abort_flag : 0;
          if (__shfl_sync(0xffffffffu, aborted, 0)) break;
        }
      }
      if (warp == 0 && lane == 0) {
        umma_commit(&fin);
        spin(&fin, 0);
        if (blockIdx.x == 0) out[0] = (clock64() - t0) / count;
      }
    } else if (staged && warp == (layout == 0 ? 3 : 12)) {
      // stands in for the TMA producer: waits for a stage to be free and marks it filled
      if (lane == 0) {
        for (int it = 0; it < count; ++it) {
          bool got = it < 4;
          for (long long n = 0; !got && n < 2000000LL; ++n) got = mbar_try(&empty[it & 3], ((it >> 2) & 1) ^ 1);
          if (!got) break;
          mbar_arrive(&full[it & 3]);
        }
      }
    } else if (warp >= 4 && warp < 12) {
      const int half = (warp - 4) >> 2;
      bool failed = false;  // after a wait gave up nothing waits any more, but every arrival still happens
      long long polls = 0, poll_cycles = 0;
      float acc[32];  // (few registers: 13 warps leave 152 per thread)
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;
      // features bit 2: two scales per K block from global memory, fetched four K blocks ahead
      const float* row_scale = scales + ((size_t)blockIdx.x * 128 + (warp & 3) * 32 + lane) * 64;
      float sa[4] = {1.f, 1.f, 1.f, 1.f}, sb[4] = {1.f, 1.f, 1.f, 1.f}, na[4], nb[4];
      for (int u = 0; u < pairs; ++u) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int j = 2 * b + half;
          const int kb = 2 * u + b;
          if ((features & 4) && (kb & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              na[i] = row_scale[(kb + 4 + i) & 63];
              nb[i] = scales[(kb + 4 + i) & 63];
            }
          }
          const float sc = (features & 4) ? sa[kb & 3] * sb[kb & 3] : 1.0001f;
          if (lane == 0 && !failed) {
            const long long c0 = clock64();
            long long n = 0;
            for (; n < 100000000LL; ++n)
              if (mbar_test(&bar[j], u & 1)) break;
            failed = n >= 100000000LL;
            polls += n + 1;
            poll_cycles += clock64() - c0;
          }
          __syncwarp();
          tc_fence_after_sync();
          if (epilogue >= 1) {
            uint32_t ra[32], rb[32];
            const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + j * 128;
            tmem_ld_32x32(taddr, ra);
            tmem_ld_32x32(taddr + 32, rb);
            tmem_ld_wait();
            if (epilogue >= 2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                acc[i] = fmaf(sc, __uint_as_float(ra[i]), acc[i]);
                acc[i] = fmaf(sc, __uint_as_float(rb[i]), acc[i]);
              }
            } else {
              acc[0] += sc * (__uint_as_float(ra[0]) + __uint_as_float(rb[0]));
            }
            tmem_ld_32x32(taddr + 64, ra);
            tmem_ld_32x32(taddr + 96, rb);
            tmem_ld_wait();
            if (epilogue >= 2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                acc[i] = fmaf(sc, __uint_as_float(ra[i]), acc[i]);
                acc[i] = fmaf(sc, __uint_as_float(rb[i]), acc[i]);
              }
            } else {
              acc[1] += sc * (__uint_as_float(ra[0]) + __uint_as_float(rb[0]));
            }
          } else {
            acc[0] += sc;
          }
          tc_fence_before_sync();
          __syncwarp();
          if (u + 1 < pairs) named_arrive(1 + j, 160);
          if ((features & 4) && (kb & 3) == 3) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              sa[i] = na[i];
              sb[i] = nb[i];
            }
          }
        }
      }
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) s += acc[i];
      if (s == 123.456f) out[7] = 1;
      if (blockIdx.x == 0 && warp == 4 && lane == 0) {
        out[1] = polls;
        out[2] = poll_cycles;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

int main() {
  long long* out;
  if (cudaMalloc(&out, 64) != cudaSuccess) return 1;
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 51200);
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  float* scales;  // features bit 2: 64 K blocks of scales for every row of every CTA (all ones)
  const size_t n_scales = (size_t)sms * 128 * 64;
  if (cudaMalloc(&scales, n_scales * sizeof(float)) != cudaSuccess) return 1;
  {
    float* ones = new float[n_scales];
    for (size_t i = 0; i < n_scales; ++i) ones[i] = 1.0f;
    cudaMemcpy(scales, ones, n_scales * sizeof(float), cudaMemcpyHostToDevice);
    delete[] ones;
  }
  long long h[8];
  auto run = [&](int mode, int count, int narrow, int layout, int epilogue, int features = 0) {
    cudaMemset(out, 0, 64);
    probe<<<sms, 416, 51200>>>(mode, count, narrow, layout, epilogue, features, scales, out);
    const cudaError_t e = cudaDeviceSynchronize();
    cudaMemcpy(h, out, 64, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) printf("error: %s\n", cudaGetErrorString(e));
    return h[0];
  };
  printf("issue rate, one thread, back to back: %lld cycles per K block (N=256), %lld (two N=128 halves); 512 = 4 x 128\n",
         run(0, 4000, 0, 0, 0), run(0, 4000, 1, 0, 0));
  for (int k : {1, 4, 8, 16})
    printf("latency: %2d multiplications (128 x 128 x 32) + commit until a polling thread sees the barrier: %lld cycles\n", k,
           run(1, k, 0, 0, 0));
  const char* layouts[3] = {"2 issuers x 2 slabs", "4 issuers x 1 slab", "1 issuer x 4 slabs"};
  const char* epilogues[3] = {"empty", "reads the slab", "reads + 128 multiply-adds per thread"};
  for (int layout = 0; layout < 3; ++layout)
    for (int epilogue = 0; epilogue < 3; ++epilogue) {
      const long long cycles = run(2, 4000, 0, layout, epilogue);
      printf("ring, %s, epilogue %s: %lld cycles per K block (two slabs) | a probe of the barrier: %.0f cycles, %.1f per wait\n",
             layouts[layout], epilogues[epilogue], cycles, h[1] ? (double)h[2] / (double)h[1] : 0.0,
             (double)h[1] / 4000.0);
    }
  // what the GEMM's loop has on top of the ring, one at a time and together (2 issuers x 2 slabs)
  const char* names[8] = {"ring alone", "+ operand stages (full/empty barriers, a stand-in producer)", "+ abort flag read by the issuers",
                          "+ stages + abort flag", "+ scales from global memory", "+ stages + scales", "+ abort flag + scales",
                          "+ stages + abort flag + scales"};
  for (int layout = 0; layout < 2; ++layout)
    for (int epilogue = 0; epilogue < 3; epilogue += 2)
      for (int features = 0; features < 8; ++features) {
        const long long cycles = run(2, 4000, 0, layout, epilogue, features);
        printf("%s, epilogue %s, %s: %lld cycles per K block | a probe of the barrier: %.0f cycles, %.1f per wait\n",
               layouts[layout], epilogue ? "reads + multiply-adds" : "empty", names[features], cycles,
               h[1] ? (double)h[2] / (double)h[1] : 0.0, (double)h[1] / 4000.0);
      }
  cudaFree(scales);
  cudaFree(out);
  return 0;
}
