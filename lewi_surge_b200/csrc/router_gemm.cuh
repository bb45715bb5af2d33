// Router projection: logits[T,E] (f32) = x[T,d] (bf16) . W[d,E] (f32) + bias, f32 FMA accumulation.
// Kept on the CUDA cores in full float32: the top-k that follows is decided by differences of a few
// ulps, so the inputs are not rounded to a tensor-core format here.
#pragma once

#include "common.cuh"

namespace lewi {

constexpr int kRgTile = 64;   // tokens x experts per CTA
constexpr int kRgK = 32;

__global__ void __launch_bounds__(256) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const float* __restrict__ w,
                                                            const float* __restrict__ bias,
                                                            float* __restrict__ logits, long long T, int d, int E) {
  __shared__ float xs[kRgK][kRgTile + 1];  // [k][token]
  __shared__ float ws[kRgK][kRgTile];      // [k][expert]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long t0 = (long long)blockIdx.x * kRgTile;
  const int e0 = blockIdx.y * kRgTile;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < d; k0 += kRgK) {
    for (int i = threadIdx.x; i < kRgTile * kRgK; i += 256) {
      const int tok = i / kRgK, kk = i % kRgK;
      const long long t = t0 + tok;
      xs[kk][tok] = (t < T && k0 + kk < d) ? __bfloat162float(x[t * d + k0 + kk]) : 0.f;
    }
    for (int i = threadIdx.x; i < kRgTile * kRgK; i += 256) {
      const int kk = i / kRgTile, ee = i % kRgTile;
      ws[kk][ee] = (k0 + kk < d && e0 + ee < E) ? w[(long long)(k0 + kk) * E + e0 + ee] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kRgK; ++kk) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + tx * 4 + j;
      if (e < E) logits[t * E + e] = acc[i][j] + (bias ? bias[e] : 0.f);
    }
  }
}

}  // namespace lewi
