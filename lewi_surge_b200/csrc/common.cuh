// Shared definitions for the MoE hot-path kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lewi_moe.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "these kernels are written for sm_100a only"
#endif

namespace lewi {

constexpr int kWarp = 32;
constexpr int kNumSMsDefault = 148;

// Per-device status word.  Kernels OR bits into it; lewi_last_status() reads and clears it.
__device__ int g_status = 0;

__device__ __forceinline__ void raise_status(int bit) { atomicOr(&g_status, bit); }

struct alignas(16) U4 {
  uint32_t x, y, z, w;
};

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Two floats -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void st_cs_v4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

inline int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kNumSMsDefault;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMsDefault;
    cached[dev] = n;
  }
  return cached[dev];
}

// Host-side count of kernel launches made through this library (read by lewi_launch_count()).
inline long long& launch_counter() {
  static long long n = 0;
  return n;
}

#define LEWI_CHECK_LAUNCH()                                 \
  do {                                                      \
    if (cudaPeekAtLastError() != cudaSuccess) {             \
      (void)cudaGetLastError();                             \
      return LEWI_ERR_CUDA;                                 \
    }                                                       \
    ++::lewi::launch_counter();                             \
  } while (0)

}  // namespace lewi
