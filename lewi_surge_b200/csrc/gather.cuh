// Row-gather kernels: the only data movement of dispatch / combine and of their gradients.
// One warp owns one output row; every lane moves 16-byte pieces, so a 2 KB bf16 row is four
// independent 128-bit loads per lane and the whole warp's traffic is fully coalesced.
// Semantics follow gather_rows / gather_reduce / gather_dot of the reference
// (modal/moe_permute.py:116-158, 161-225, 228-234): multiply and accumulate in float32.
#pragma once

#include "common.cuh"

namespace lewi {

constexpr int kGatherThreads = 256;

template <typename T>
struct Elem;  // 16-byte vector <-> 4 or 8 floats

template <>
struct Elem<float> {
  static constexpr int kPerVec = 4;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
};

// out[i] = x[src(i)] * scale.  VPL = 16-byte vectors per lane (row bytes <= VPL*512).
template <typename T, int VPL>
__global__ void __launch_bounds__(kGatherThreads) gather_rows_kernel(
    const T* __restrict__ x, const int32_t* __restrict__ idx, const float* __restrict__ scale, T* __restrict__ out,
    long long n_src, long long m, int d, int idx_div, int scale_by_idx, const int32_t* __restrict__ n_rows_dev,
    int rows_per_unit) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  long long rows = m;
  if (n_rows_dev != nullptr) rows = min(rows, (long long)n_rows_dev[0] * rows_per_unit);
  const int nvec = d / Elem<T>::kPerVec;
  for (long long i = warp0; i < rows; i += n_warps) {
    const int raw = idx[i];
    long long src = raw;
    if (idx_div > 1 && raw >= 0) src = raw / idx_div;
    const bool zero = raw < 0;
    if (!zero && src >= n_src) {
      if (lane == 0) raise_status(LEWI_STATUS_BAD_INDEX);
      continue;
    }
    uint4 v[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      int vi = lane + c * kWarp;
      v[c] = make_uint4(0, 0, 0, 0);
      if (!zero && vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(x + src * d) + vi);
    }
    if (scale != nullptr && !zero) {
      const float s = scale[scale_by_idx ? (long long)raw : i];
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        float f[Elem<T>::kPerVec];
        Elem<T>::unpack(v[c], f);
#pragma unroll
        for (int q = 0; q < Elem<T>::kPerVec; ++q) f[q] *= s;
        v[c] = Elem<T>::pack(f);
      }
    }
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      int vi = lane + c * kWarp;
      if (vi < nvec) st_v4(reinterpret_cast<uint4*>(out + i * d) + vi, v[c]);
    }
  }
}

// Dispatch in token order: out[pos[t,j]] = x[t] for the k slots of token t; padded rows that hold no slot
// (row_slot[r] < 0) become zero rows.  Every output row has exactly one writer, so this is the same function as
// the row gather out[r] = x[row_slot[r] / k] -- but each source row is read once instead of k times at k distant
// moments, which keeps the read side at T rows of DRAM traffic however large the source is against the L2.
template <int VPL>
__global__ void __launch_bounds__(kGatherThreads) dispatch_rows_kernel(
    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ pos, const int32_t* __restrict__ row_slot,
    __nv_bfloat16* __restrict__ out, long long n_tokens, int k, int d, long long out_rows,
    const int32_t* __restrict__ n_rows_dev, int rows_per_unit) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  long long rows = out_rows;
  if (n_rows_dev != nullptr) rows = min(rows, (long long)n_rows_dev[0] * rows_per_unit);
  for (long long t = warp0; t < n_tokens; t += n_warps) {
    const int my_pos = lane < k ? pos[t * k + lane] : -1;
    uint4 v[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      v[c] = make_uint4(0, 0, 0, 0);
      if (vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(x + t * d) + vi);
    }
    for (int j = 0; j < k; ++j) {
      const long long p = __shfl_sync(0xffffffffu, my_pos, j);
      if (p < 0 || p >= rows) {
        if (lane == 0 && p >= rows) raise_status(LEWI_STATUS_BAD_INDEX);
        continue;
      }
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int vi = lane + c * kWarp;
        if (vi < nvec) st_v4(reinterpret_cast<uint4*>(out + p * d) + vi, v[c]);
      }
    }
  }
  // zero rows of the padded layout
  for (long long r0 = warp0 * kWarp; r0 < rows; r0 += n_warps * kWarp) {
    const long long r = r0 + lane;
    const unsigned empty = __ballot_sync(0xffffffffu, r < rows && row_slot[r] < 0);
    for (unsigned m = empty; m != 0; m &= m - 1) {
      const long long rr = r0 + (__ffs(m) - 1);
      for (int vi = lane; vi < nvec; vi += kWarp) st_v4(reinterpret_cast<uint4*>(out + rr * d) + vi, make_uint4(0, 0, 0, 0));
    }
  }
}

// out[t] = sum_j w[t,j] * y[pos[t,j]] (+ add0[t] + add1[t]); f32 accumulate.
template <typename TI, typename TO, int VPL>
__global__ void __launch_bounds__(kGatherThreads) gather_reduce_kernel(
    const TI* __restrict__ y, const int32_t* __restrict__ pos, const float* __restrict__ w,
    const TI* __restrict__ add0, const TI* __restrict__ add1, TO* __restrict__ out, long long n, int k, int d,
    long long n_y_rows) {
  constexpr int PV = Elem<TI>::kPerVec;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / PV;
  for (long long t = warp0; t < n; t += n_warps) {
    float acc[VPL][PV];
#pragma unroll
    for (int c = 0; c < VPL; ++c)
#pragma unroll
      for (int q = 0; q < PV; ++q) acc[c][q] = 0.f;
    int my_pos = 0;
    float my_w = 1.f;
    if (lane < k) {
      my_pos = pos[t * k + lane];
      if (w != nullptr) my_w = w[t * k + lane];
    }
    for (int j = 0; j < k; ++j) {
      const long long p = __shfl_sync(0xffffffffu, my_pos, j);
      const float wj = __shfl_sync(0xffffffffu, my_w, j);
      if (p < 0 || p >= n_y_rows) {
        if (lane == 0 && p >= n_y_rows) raise_status(LEWI_STATUS_BAD_INDEX);
        continue;
      }
      uint4 v[VPL];
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        int vi = lane + c * kWarp;
        v[c] = make_uint4(0, 0, 0, 0);
        if (vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(y + p * d) + vi);
      }
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        float f[PV];
        Elem<TI>::unpack(v[c], f);
#pragma unroll
        for (int q = 0; q < PV; ++q) acc[c][q] = fmaf(wj, f[q], acc[c][q]);
      }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const TI* add = a == 0 ? add0 : add1;
      if (add == nullptr) continue;
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        int vi = lane + c * kWarp;
        if (vi < nvec) {
          float f[PV];
          Elem<TI>::unpack(ld_nc_v4(reinterpret_cast<const uint4*>(add + t * d) + vi), f);
#pragma unroll
          for (int q = 0; q < PV; ++q) acc[c][q] += f[q];
        }
      }
    }
    // store: PV input elements per vector -> PV output elements
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      int vi = lane + c * kWarp;
      if (vi >= nvec) continue;
      TO* o = out + t * d + (long long)vi * PV;
      if constexpr (sizeof(TO) == 4) {
#pragma unroll
        for (int q = 0; q < PV; q += 4) st_v4(reinterpret_cast<float*>(o) + q, Elem<float>::pack(&acc[c][q]));
      } else {
        if constexpr (PV == 8) {
          st_v4(o, Elem<__nv_bfloat16>::pack(acc[c]));
        } else {
          uint2 pk = make_uint2(pack_bf16(acc[c][0], acc[c][1]), pack_bf16(acc[c][2], acc[c][3]));
          *reinterpret_cast<uint2*>(o) = pk;
        }
      }
    }
  }
}

// out[t,j] = <g[t], y[pos[t,j]]>.
template <typename T, int VPL>
__global__ void __launch_bounds__(kGatherThreads) gather_dot_kernel(
    const T* __restrict__ y, const int32_t* __restrict__ pos, const T* __restrict__ g, float* __restrict__ out,
    long long n, int k, int d, long long n_y_rows) {
  constexpr int PV = Elem<T>::kPerVec;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / PV;
  for (long long t = warp0; t < n; t += n_warps) {
    float gv[VPL][PV];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      int vi = lane + c * kWarp;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (vi < nvec) v = ld_nc_v4(reinterpret_cast<const uint4*>(g + t * d) + vi);
      Elem<T>::unpack(v, gv[c]);
    }
    int my_pos = (lane < k) ? pos[t * k + lane] : 0;
    float my_out = 0.f;
    for (int j = 0; j < k; ++j) {
      const long long p = __shfl_sync(0xffffffffu, my_pos, j);
      float s = 0.f;
      if (p >= 0 && p < n_y_rows) {
#pragma unroll
        for (int c = 0; c < VPL; ++c) {
          int vi = lane + c * kWarp;
          if (vi < nvec) {
            float f[PV];
            Elem<T>::unpack(ld_nc_v4(reinterpret_cast<const uint4*>(y + p * d) + vi), f);
#pragma unroll
            for (int q = 0; q < PV; ++q) s = fmaf(gv[c][q], f[q], s);
          }
        }
      } else if (lane == 0 && p >= n_y_rows) {
        raise_status(LEWI_STATUS_BAD_INDEX);
      }
      s = warp_sum(s);
      if (lane == j) my_out = s;
    }
    if (lane < k) out[t * k + lane] = my_out;
  }
}

inline int gather_grid(long long rows) {
  const long long warps_per_cta = kGatherThreads / kWarp;
  long long ctas = (rows + warps_per_cta - 1) / warps_per_cta;
  const long long cap = (long long)num_sms() * 16;  // 8 resident CTAs per SM x 2 waves
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  return (int)ctas;
}

// smallest supported VPL in {1,2,4,8,16} covering the row, or 0
inline int pick_vpl(int d, int elem_bytes) {
  const long long row_bytes = (long long)d * elem_bytes;
  if (row_bytes % 16 != 0) return 0;
  const long long nvec = row_bytes / 16;
  for (int v = 1; v <= 16; v *= 2)
    if (nvec <= (long long)v * kWarp) return v;
  return 0;
}

#define LEWI_DISPATCH_VPL(VPL_VALUE, ...)        \
  switch (VPL_VALUE) {                           \
    case 1: { constexpr int VPL = 1; __VA_ARGS__; } break;   \
    case 2: { constexpr int VPL = 2; __VA_ARGS__; } break;   \
    case 4: { constexpr int VPL = 4; __VA_ARGS__; } break;   \
    case 8: { constexpr int VPL = 8; __VA_ARGS__; } break;   \
    default: { constexpr int VPL = 16; __VA_ARGS__; } break; \
  }

}  // namespace lewi
