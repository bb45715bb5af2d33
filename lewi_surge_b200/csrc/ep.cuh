// Expert-parallel dispatch / combine as kernels over peer memory (NVLink loads and stores).
//
// Rank g owns experts [g*El, (g+1)*El).  After the ranks have exchanged their expert histograms
// (counts_all [G,E], a tiny all-gather), every rank can compute where its rows live on the owner:
//   owner layout   rows of local expert el from all sources, source-major inside the expert, each expert
//                  padded to a multiple of 128 rows (the layout the grouped GEMMs consume);
//   dst_base[e]    first row, in the owner's buffer, of THIS rank's rows for global expert e.
// Dispatch is then one gather kernel whose stores go straight into the owners' buffers, and combine is
// one gather-reduce kernel whose loads come straight from the owners' outputs: no send/receive staging,
// no re-sort on arrival.  Nothing here waits on another GPU; ordering between ranks is done with
// stream-ordered collectives by the host code.  Plain loads/stores only (no multimem, no TMA).
#pragma once

#include "common.cuh"
#include "gather.cuh"
#include "routing.cuh"

namespace lewi {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

// One CTA.  counts_all [G,E]; outputs as described above.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ counts_all, int G, int E, int me,
                                                       int block, long long rmax_pad, int nbmax,
                                                       int32_t* dst_base, int32_t* pad_offsets, int32_t* valid_end,
                                                       int32_t* n_blocks, int32_t* block_expert,
                                                       int32_t* recv_rows) {
  __shared__ int s_total[kMaxExperts];   // rows of expert e over all sources
  __shared__ int s_before[kMaxExperts];  // rows of expert e from sources < me
  __shared__ int s_pad[kMaxExperts + 1]; // padded start of expert e on ITS owner
  const int El = E / G;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, bef = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts_all[s * E + e];
      tot += c;
      if (s < me) bef += c;
    }
    s_total[e] = tot;
    s_before[e] = bef;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / El) * El;   // first expert of e's owner
    int pad = 0;
    for (int x = first; x < e; ++x) pad += (s_total[x] + block - 1) / block * block;
    s_pad[e] = pad;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst_base[e] = s_pad[e] + s_before[e];
  // this rank as owner
  const int e0 = me * El;
  for (int el = threadIdx.x; el <= El; el += blockDim.x) {
    int v;
    if (el < El) {
      v = s_pad[e0 + el];
      valid_end[el] = v + s_total[e0 + el];
    } else {
      const int last = e0 + El - 1;
      v = s_pad[last] + (s_total[last] + block - 1) / block * block;
    }
    pad_offsets[el] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int last = e0 + El - 1;
    const long long total_pad = s_pad[last] + (s_total[last] + block - 1) / block * block;
    if (total_pad > rmax_pad) raise_status(LEWI_STATUS_EP_OVERFLOW);
    n_blocks[0] = (int)(min(total_pad, rmax_pad) / block);
    int rows = 0;
    for (int el = 0; el < El; ++el) rows += s_total[e0 + el];
    recv_rows[0] = rows;
  }
  if (block_expert != nullptr) {
    const int last = e0 + El - 1;
    const int nb = (s_pad[last] + (s_total[last] + block - 1) / block * block) / block;
    for (int b = threadIdx.x; b < nbmax; b += blockDim.x) {
      int val = -1;
      if (b < nb) {
        const int row = b * block;
        int lo = 0, hi = El;
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (s_pad[e0 + mid] <= row) lo = mid; else hi = mid;
        }
        val = lo;
      }
      block_expert[b] = val;
    }
  }
}

// Dispatch: sorted position p of this rank (slot order[p], token order[p]/k, expert e) goes to row
// dst_base[e] + (p - offsets[e]) of the owner's buffer.  One warp per row; also records, per slot,
// the owner and the row for the later pulls, and optionally pushes the slot's router weight.
template <int VPL>
__global__ void __launch_bounds__(kGatherThreads) ep_push_rows_kernel(
    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ order, const int32_t* __restrict__ flat_expert,
    const int32_t* __restrict__ offsets, const int32_t* __restrict__ dst_base, const float* __restrict__ slot_w,
    PeerPtrs peer_rows, PeerPtrs peer_w, int32_t* __restrict__ slot_rank, int32_t* __restrict__ slot_row,
    long long m, int k, int d, int El, int G, long long rmax_pad, long long n_tokens) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  for (long long p = warp0; p < m; p += n_warps) {
    const int slot = order[p];
    const int e = flat_expert[slot];
    const long long tok = slot / k;
    if (e < 0 || e >= El * G || tok >= n_tokens) {
      if (lane == 0) raise_status(LEWI_STATUS_BAD_INDEX);
      continue;
    }
    const int r = e / El;
    const long long row = (long long)dst_base[e] + (p - offsets[e]);
    if (lane == 0 && slot_rank != nullptr) {
      slot_rank[slot] = r;
      slot_row[slot] = (int)row;
    }
    if (row >= rmax_pad) continue;   // capacity overflow: reported by the plan kernel
    uint4 v[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      v[c] = make_uint4(0, 0, 0, 0);
      if (vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(x + tok * d) + vi);
    }
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peer_rows.p[r]) + row * d;
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      if (vi < nvec) st_v4(reinterpret_cast<uint4*>(dst) + vi, v[c]);
    }
    if (lane == 0 && slot_w != nullptr) reinterpret_cast<float*>(peer_w.p[r])[row] = slot_w[slot];
  }
}

// Owner side: the unused tail of every expert's last block must be zero rows.
__global__ void __launch_bounds__(256) ep_zero_pad_kernel(__nv_bfloat16* buf, const int32_t* __restrict__ valid_end,
                                                          const int32_t* __restrict__ pad_offsets, int d,
                                                          long long rmax_pad) {
  const int el = blockIdx.x;
  const long long r0 = valid_end[el], r1 = min((long long)pad_offsets[el + 1], rmax_pad);
  const long long n16 = (r1 > r0 ? (r1 - r0) : 0) * d / 8;
  uint4* base = reinterpret_cast<uint4*>(buf + r0 * d);
  for (long long i = threadIdx.x; i < n16; i += blockDim.x) base[i] = make_uint4(0, 0, 0, 0);
}

// Combine: out[t] = sum_j peer[slot_rank[t,j]][slot_row[t,j]] (+ add0[t] + add1[t]); loads cross NVLink.
template <int VPL>
__global__ void __launch_bounds__(kGatherThreads) ep_pull_reduce_kernel(
    PeerPtrs peer_rows, const int32_t* __restrict__ slot_rank, const int32_t* __restrict__ slot_row,
    const __nv_bfloat16* __restrict__ add0, const __nv_bfloat16* __restrict__ add1, __nv_bfloat16* __restrict__ out,
    long long n, int k, int d, int G, long long rmax_pad) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  for (long long t = warp0; t < n; t += n_warps) {
    float acc[VPL][8];
#pragma unroll
    for (int c = 0; c < VPL; ++c)
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[c][q] = 0.f;
    int my_rank = 0, my_row = -1;
    if (lane < k) {
      my_rank = slot_rank[t * k + lane];
      my_row = slot_row[t * k + lane];
    }
    for (int j = 0; j < k; ++j) {
      const int r = __shfl_sync(0xffffffffu, my_rank, j);
      const long long row = __shfl_sync(0xffffffffu, my_row, j);
      if (r < 0 || r >= G || row < 0 || row >= rmax_pad) continue;
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(peer_rows.p[r]) + row * d;
      uint4 v[VPL];
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int vi = lane + c * kWarp;
        v[c] = make_uint4(0, 0, 0, 0);
        if (vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(src) + vi);
      }
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        float f[8];
        Elem<__nv_bfloat16>::unpack(v[c], f);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[c][q] += f[q];
      }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const __nv_bfloat16* add = a == 0 ? add0 : add1;
      if (add == nullptr) continue;
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int vi = lane + c * kWarp;
        if (vi < nvec) {
          float f[8];
          Elem<__nv_bfloat16>::unpack(ld_nc_v4(reinterpret_cast<const uint4*>(add + t * d) + vi), f);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[c][q] += f[q];
        }
      }
    }
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      if (vi < nvec) st_v4(reinterpret_cast<uint4*>(out + t * d) + vi, Elem<__nv_bfloat16>::pack(acc[c]));
    }
  }
}

// Routing-weight gradient: dw[slot] = sum_p peer_partial[slot_rank][slot_row * parts + p].
__global__ void __launch_bounds__(256) ep_pull_dw_kernel(PeerPtrs peer_partial, const int32_t* __restrict__ slot_rank,
                                                         const int32_t* __restrict__ slot_row, float* __restrict__ dw,
                                                         long long m, int parts, int G, long long rmax_pad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (long long)gridDim.x * blockDim.x) {
    const int r = slot_rank[i];
    const long long row = slot_row[i];
    float s = 0.f;
    if (r >= 0 && r < G && row >= 0 && row < rmax_pad) {
      const float* src = reinterpret_cast<const float*>(peer_partial.p[r]) + row * parts;
      for (int p = 0; p < parts; ++p) s += src[p];
    }
    dw[i] = s;
  }
}

}  // namespace lewi
