// Host-side helpers shared by the C-ABI entry points: status codes, the driver
// entry point used to encode TMA tensor maps (fetched at run time so the library
// links against the CUDA runtime only) and a per-device SM count cache.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Return codes of every extern "C" entry point (see include/b200moe.h).
enum : int {
  B200MOE_OK = 0,
  B200MOE_ERR_ARG = -1,        // null pointer, negative size, unsupported combination
  B200MOE_ERR_ALIGN = -2,      // pointer / pitch alignment requirement not met
  B200MOE_ERR_TENSORMAP = -3,  // cuTensorMapEncodeTiled refused the operand
  B200MOE_ERR_LAUNCH = -4,     // kernel launch failed (cudaGetLastError != success)
  B200MOE_ERR_DRIVER = -5,     // driver entry point unavailable
  B200MOE_ERR_LIMIT = -6       // size beyond a documented maximum
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled();
int sm_count_device();      // SM count of the current device (cached per device)
int sm_count();             // CTAs a persistent kernel may launch: the SM count, or the limit below
void set_cta_limit(int n);  // n > 0: persistent kernels launch at most n CTAs; 0: no limit

// Encodes a row-major tensor of `rank` dims.  dims[0] is the innermost (contiguous)
// extent in elements; strides_bytes[i] is the byte pitch of dims[i+1].
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_LAUNCH; }

}  // namespace b200
